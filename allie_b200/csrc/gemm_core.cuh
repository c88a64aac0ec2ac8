// Device-side pieces shared by the tcgen05 GEMM kernels (gemm_tc.cu: plain and CTA-pair kernels;
// gemm_grouped.cu: the grouped CTA-pair kernel of the MoE expert layers): tile constants, the
// kernel argument block, the fused epilogue math and the routines with which an epilogue warp
// drains its part of a finished accumulator.
#pragma once
#include "gemm_tc.cuh"
#include "ptx.cuh"

namespace ab {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_EPI_WARPS = 16;
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;

// CTA-pair kernels (cta_group::2, 256 x 256 tiles)
constexpr int PAIR_STAGES = 5;
constexpr int PAIR_WARP_STAGING = 4096;   // one wide staging tile per epilogue warp
constexpr int PAIR_BN = 256;      // instruction N; each CTA stages PAIR_BN / 2 columns of B

struct GemmArgs {
  int M, N, K;
  int k_splits;
  int pdl;            // launched as a programmatic dependent: B (weights) may be fetched before griddep_wait
  int aux_tma;        // act == 2 in the CTA-pair kernel: the aux tile of an epilogue warp arrives by TMA in
                      // the warp's staging tile (tmAux is a load map) instead of by row loads
  AbGemmEpilogue ep;
  const unsigned long long* salt;   // seed_salt_ptr() at launch: folded into ep.drop_seed when not null
  int* status;
};

// Fused epilogue math for 8 adjacent columns n..n+7 of row m.  `v` comes in as the raw fp32
// accumulators and leaves as the final values; `pre` receives the bf16 pre-activation when
// act == 1.  Reads (bias, aux for act == 2, residual) are predicated by the caller's `ok`.
// `bias_off` shifts the bias vector (grouped GEMMs: one bias row per group).
__device__ __forceinline__ void epilogue_math8(const GemmArgs& g, float* v, uint4& pre, int m, int n,
                                               bool ok, bool add_bias, int bias_off = 0,
                                               const uint4* aux_staged = nullptr) {
  const AbGemmEpilogue& ep = g.ep;
  if (ep.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= ep.alpha;
  }
  if (!ok) return;
  if (ep.bias && add_bias) {      // with split-K only the first split carries the bias
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(ep.bias + bias_off + n));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(ep.bias + bias_off + n + 4));
    v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
    v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
  }
  if (ep.act == 1 && ep.aux_grad) {
    // the second output is gelu'(pre-activation): the backward epilogue only multiplies by it
    float d[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh_with_grad(v[j], d[j]);
    pre.x = pack_bf16x2(d[0], d[1]); pre.y = pack_bf16x2(d[2], d[3]);
    pre.z = pack_bf16x2(d[4], d[5]); pre.w = pack_bf16x2(d[6], d[7]);
  } else if (ep.act == 1) {
    pre.x = pack_bf16x2(v[0], v[1]); pre.y = pack_bf16x2(v[2], v[3]);
    pre.z = pack_bf16x2(v[4], v[5]); pre.w = pack_bf16x2(v[6], v[7]);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
  } else if (ep.act == 3) {        // GELU without keeping the pre-activation (inference)
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
  } else if (ep.act == 2) {
    // the eight aux values: from the staged tile in shared memory, or straight from global
    const uint4 q = aux_staged ? *aux_staged
                               : *reinterpret_cast<const uint4*>(
                                     static_cast<const __nv_bfloat16*>(ep.aux) + (long long)m * ep.ldaux + n);
    if (ep.aux_grad) {        // aux already holds the derivative (written by an act == 1 launch with aux_grad)
      v[0] *= bf16_lo(q.x); v[1] *= bf16_hi(q.x); v[2] *= bf16_lo(q.y); v[3] *= bf16_hi(q.y);
      v[4] *= bf16_lo(q.z); v[5] *= bf16_hi(q.z); v[6] *= bf16_lo(q.w); v[7] *= bf16_hi(q.w);
    } else {
    v[0] *= gelu_tanh_grad(bf16_lo(q.x)); v[1] *= gelu_tanh_grad(bf16_hi(q.x));
    v[2] *= gelu_tanh_grad(bf16_lo(q.y)); v[3] *= gelu_tanh_grad(bf16_hi(q.y));
    v[4] *= gelu_tanh_grad(bf16_lo(q.z)); v[5] *= gelu_tanh_grad(bf16_hi(q.z));
    v[6] *= gelu_tanh_grad(bf16_lo(q.w)); v[7] *= gelu_tanh_grad(bf16_hi(q.w));
    }
  }
  if (ep.resid) {
    if (ep.drop_thr16) {
      const uint64_t group = (static_cast<uint64_t>(m) * g.N + n) >> 3;
      const uint32_t keep = dropout_keep8(salted(ep.drop_seed, g.salt), ep.drop_stream, group, ep.drop_thr16);
      const float s = dropout_scale(ep.drop_thr16);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = ((keep >> j) & 1u) ? v[j] * s : 0.f;
    }
    const float4 r0 = *reinterpret_cast<const float4*>(ep.resid + (long long)m * ep.ldr + n);
    const float4 r1 = *reinterpret_cast<const float4*>(ep.resid + (long long)m * ep.ldr + n + 4);
    v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
    v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
  }
}

// One epilogue warp drains its 32 rows x COLS columns of a finished accumulator: TMEM -> registers
// -> fused math -> swizzled staging tile -> TMA store (or reduce-add), 16 columns per round.
template <int COLS>
__device__ __forceinline__ void epilogue_drain(const GemmArgs& g, const CUtensorMap& tmOut,
                                               const CUtensorMap& tmAux, uint32_t taddr, int m,
                                               int m0w, int nbase, bool row_ok, uint8_t* my_stage,
                                               int lane, bool add_bias) {
#pragma unroll 1
  for (int rd = 0; rd < COLS / 16; ++rd) {      // rounds of 16 columns
    const int n0 = nbase + rd * 16;
    if (n0 >= g.N) break;                                 // warp-uniform
    uint32_t r[16];
    tmem_ld16(taddr + rd * 16, r);
    if (lane == 0) tma_store_wait_read<0>();              // staging tile free again
    __syncwarp();
    tmem_ld_wait();
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      const int n = n0 + grp * 8;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[grp * 8 + j]);
      uint4 pre = make_uint4(0, 0, 0, 0);
      epilogue_math8(g, v, pre, m, n, row_ok && n < g.N, add_bias);
      if (g.ep.out_fp32) {
        // 16 fp32 columns = 64-byte rows, 64B swizzle: 16-byte chunk index ^= (row >> 1) & 3
        uint8_t* rowp = my_stage + lane * 64;
        const int sw = (lane >> 1) & 3;
        *reinterpret_cast<float4*>(rowp + (((2 * grp) ^ sw) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(rowp + (((2 * grp + 1) ^ sw) << 4)) = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        // 16 bf16 columns = 32-byte rows, 32B swizzle: chunk index ^= (row >> 2) & 1
        const uint32_t off = lane * 32 + ((grp ^ ((lane >> 2) & 1)) << 4);
        uint4 o;
        o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(my_stage + off) = o;
        if (g.ep.act == 1) *reinterpret_cast<uint4*>(my_stage + 1024 + off) = pre;
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (g.ep.accumulate) tma_reduce_add_2d(&tmOut, my_stage, n0, m0w);
      else                 tma_store_2d(&tmOut, my_stage, n0, m0w);
      if (g.ep.act == 1) tma_store_2d(&tmAux, my_stage + 1024, n0, m0w);
      tma_store_commit();
    }
  }
}

// Drain used by the CTA-pair kernel: the same per-round math, but several 16-column rounds are
// staged side by side in one 4 KB tile per warp and leave in one TMA store with 128-byte rows
// (64 bf16 or 32 fp32 columns; 64-byte rows when a second bf16 output shares the tile).  Wide
// rows matter: the store path costs per row segment, not per byte.
template <int COLS>
__device__ __forceinline__ void epilogue_drain_wide(const GemmArgs& g, const CUtensorMap& tmOut,
                                                    const CUtensorMap& tmAux, uint32_t taddr, int m,
                                                    int m0w, int nbase, bool row_ok, uint8_t* stg,
                                                    int lane, bool add_bias, int bias_off = 0,
                                                    bool aux_in_stage = false) {
  // aux_in_stage (act == 2, one bf16 output, COLS == 64): the staging tile already holds the aux
  // tile in the layout of the output tile (same box, same swizzle), so a lane reads its eight aux
  // values from the very chunk it then overwrites with its eight results.
  const bool two = g.ep.act == 1, f32 = g.ep.out_fp32 != 0;
  const int gcols = (f32 || two) ? 32 : 64;             // columns per TMA store (warp-uniform)
#pragma unroll 1
  for (int g0 = 0; g0 < COLS; g0 += gcols) {
    const int gn0 = nbase + g0;
    if (gn0 >= g.N) break;                              // warp-uniform
    if (lane == 0) tma_store_wait_read<0>();            // staging tile free again
    __syncwarp();
#pragma unroll 1
    for (int rd = 0; rd < gcols / 16; ++rd) {
      const int n0 = gn0 + rd * 16;
      if (n0 >= g.N) break;
      uint32_t r[16];
      tmem_ld16(taddr + g0 + rd * 16, r);
      tmem_ld_wait();
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        const int n = n0 + grp * 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[grp * 8 + j]);
        uint4 pre = make_uint4(0, 0, 0, 0);
        const uint4* staged = aux_in_stage
            ? reinterpret_cast<const uint4*>(stg + lane * 128 + (((rd * 2 + grp) ^ (lane & 7)) << 4)) : nullptr;
        epilogue_math8(g, v, pre, m, n, row_ok && n < g.N, add_bias, bias_off, staged);
        if (f32) {
          // 32 fp32 columns = 128-byte rows, 128B swizzle: 16-byte chunk index ^= row & 7
          uint8_t* rowp = stg + lane * 128;
          const int c = rd * 4 + grp * 2, sw = lane & 7;
          *reinterpret_cast<float4*>(rowp + ((c ^ sw) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(rowp + (((c + 1) ^ sw) << 4)) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          uint4 o;
          o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
          o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
          const int c = rd * 2 + grp;
          if (two) {   // 32 bf16 columns = 64-byte rows, 64B swizzle; pre-activation tile 2 KB further
            const uint32_t off = lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(stg + off) = o;
            *reinterpret_cast<uint4*>(stg + 2048 + off) = pre;
          } else {     // 64 bf16 columns = 128-byte rows, 128B swizzle
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) = o;
          }
        }
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (g.ep.accumulate) tma_reduce_add_2d(&tmOut, stg, gn0, m0w);
      else                 tma_store_2d(&tmOut, stg, gn0, m0w);
      if (two) tma_store_2d(&tmAux, stg + 2048, gn0, m0w);
      tma_store_commit();
    }
  }
}

}  // namespace ab
