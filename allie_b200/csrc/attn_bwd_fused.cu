// Single-kernel attention backward for head_dim 64 (the medium / large configurations).
//
// A CTA owns one 128-row key/value tile j of one (batch, head) and streams the query tiles
// i >= j.  Per pair (i, j) the tensor core runs five products, S and dP into TMEM, then
// dV += P^T dO, dK += dS^T Q (accumulated over i in TMEM) and dQ_ij = dS K_j (fresh each time,
// double-buffered).  The 16 math warps turn S/dP into P/dS exactly once per pair - half the
// exponentials and dropout work of the two-kernel scheme - and push each dQ_ij tile to an fp32
// accumulator in global memory with TMA reduce-add, one 32x16 box per warp, so no atomics are
// issued by threads.  A trailing kernel converts the fp32 dQ to bf16 into the packed dQKV
// activation and clears the accumulator for the next layer.
//
// TMEM columns (512): S 0-127 | dP 128-255 | dV 256-319 | dK 320-383 | dQ 384-447, 448-511.
#include "attn_common.cuh"
#include <cstdlib>

namespace ab {


constexpr int FB_MATH_WARPS = 16;
constexpr int FB_MATH_THREADS = FB_MATH_WARPS * 32;
constexpr int FB_TMA_WARP = FB_MATH_WARPS;
constexpr int FB_MMA_WARP = FB_MATH_WARPS + 1;
constexpr int FB_THREADS = (FB_MATH_WARPS + 2) * 32;
constexpr int FB_TILE = 128 * 64 * 2;       // one 128 x 64 bf16 tile
constexpr int FB_P = 128 * 128 * 2;

// P and dS for 16 adjacent keys of one query row.
//   p_i  = exp2(s_i * sl2 - lse_l2)                       (0 on masked keys)
//   P_i  = keep_i ? p_i * dscale : 0                      (what multiplies dO in dV)
//   dS_i = p_i * ((keep_i ? dP_i * dscale : 0) - delta) * scale
// A row outside the sequence passes lse_l2 = +inf, which makes every p_i zero without a select;
// the dropout decision is applied as a multiplication by m_i = keep_i ? dscale : 0.
template <bool DIAG, bool DROP>
__device__ __forceinline__ void fb_math16(const uint32_t* sv, const uint32_t* dv, float* p, float* ds,
                                          int r, int col0, float sl2, float lse_l2,
                                          float dlt_s, float scale, float dscale, uint32_t keep16) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float pi = ex2_fast(__uint_as_float(sv[i]) * sl2 - lse_l2);
    if (DIAG) pi = (col0 + i) <= r ? pi : 0.f;
    if (DROP) {
      const float mi = ((keep16 >> i) & 1u) ? dscale : 0.f;
      p[i] = pi * mi;
      ds[i] = pi * (__uint_as_float(dv[i]) * (mi * scale) - dlt_s);
    } else {
      p[i] = pi;
      ds[i] = pi * (__uint_as_float(dv[i]) * scale - dlt_s);
    }
  }
}

__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_fused64_kernel(const __grid_constant__ CUtensorMap tmQKV,
                        const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmDQ, const AttnBwdArgs a) {
  griddep_enter();
  constexpr int HD = 64;
  constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_T = make_idesc_bf16(128, HD, 1, 1);
  constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, HD, 0, 1);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + FB_TILE;
  uint8_t* sQ = sV + FB_TILE;            // 2 stages
  uint8_t* sDO = sQ + 2 * FB_TILE;       // 2 stages
  uint8_t* sP = sDO + 2 * FB_TILE;
  uint8_t* sDS = sP + FB_P;
  uint8_t* sDQ = sDS + FB_P;             // 16 warps x 2 KB staging for the dQ reduce-adds
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDQ + FB_MATH_WARPS * 2048);
  uint64_t* stat_full = bars;
  uint64_t* full = bars + 1;       // 2
  uint64_t* empty = bars + 3;      // 2
  uint64_t* sdp_full = bars + 5;
  uint64_t* sdp_empty = bars + 6;
  uint64_t* pds_full = bars + 7;
  uint64_t* pds_empty = bars + 8;
  uint64_t* dq_full = bars + 9;    // 2
  uint64_t* dq_empty = bars + 11;  // 2
  uint64_t* acc_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (a.T + 127) / 128;
  const int h = blockIdx.y, b = blockIdx.z;
  const int own = static_cast<int>(blockIdx.x);     // key tile; small index = most query tiles first
  const int n_iter = nt - own;
  const int d_model = a.H * HD;

  if (threadIdx.x == 0) {
    mbar_init(stat_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&full[i], 1); mbar_init(&empty[i], 1);
      mbar_init(&dq_full[i], 1); mbar_init(&dq_empty[i], FB_MATH_WARPS);
    }
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, FB_MATH_WARPS);
    mbar_init(pds_full, FB_MATH_WARPS); mbar_init(pds_empty, 1); mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == FB_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 320,
                 tDQ = tmem_base + 384;

  if (warp == FB_TMA_WARP) {
    if (lane == 0) {
      const int row_own = b * a.T + own * 128;
      mbar_expect_tx(stat_full, 2 * FB_TILE);
      tma_load_2d(sK, &tmQKV, stat_full, d_model + h * HD, row_own);
      tma_load_2d(sV, &tmQKV, stat_full, 2 * d_model + h * HD, row_own);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const int row = b * a.T + (own + it) * 128;
        if (!mbar_wait(&empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break;
        }
        mbar_expect_tx(&full[st], 2 * FB_TILE);
        tma_load_2d(sQ + st * FB_TILE, &tmQKV, &full[st], h * HD, row);
        tma_load_2d(sDO + st * FB_TILE, &tmDO, &full[st], h * HD, row);
      }
    }
  } else if (warp == FB_MMA_WARP) {
    if (lane == 0) {
      bool ok = mbar_wait(stat_full, 0, abort_flag);
      const uint32_t k0 = smem_u32(sK), v0 = smem_u32(sV), p0 = smem_u32(sP), ds0 = smem_u32(sDS);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;
        if (!mbar_wait(&full[st], (it >> 1) & 1, abort_flag)) return false;
        if (it > 0 && !mbar_wait(sdp_empty, (it - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q = smem_u32(sQ + st * FB_TILE), dO = smem_u32(sDO + st * FB_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tS, make_sdesc_sw128(q + k * 32, 16, 1024), make_sdesc_sw128(k0 + k * 32, 16, 1024),
                    IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tDP, make_sdesc_sw128(dO + k * 32, 16, 1024), make_sdesc_sw128(v0 + k * 32, 16, 1024),
                    IDESC_S, k > 0);
        umma_commit(sdp_full);
        return true;
      };
      auto issue_acc = [&](int it) {
        const int st = it & 1;
        if (!mbar_wait(pds_full, it & 1, abort_flag)) return false;
        if (it >= 2 && !mbar_wait(&dq_empty[it & 1], ((it - 2) >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q = smem_u32(sQ + st * FB_TILE), dO = smem_u32(sDO + st * FB_TILE);
        // dQ_ij = dS K_j first: its consumers (the math warps) can start draining it earliest
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDQ + (it & 1) * 64, make_sdesc_sw128(ds0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                    make_sdesc_sw128(k0 + k * 2048, 16384, 1024), IDESC_DQ, k > 0);
        umma_commit(&dq_full[it & 1]);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDV, make_sdesc_sw128(p0 + k * 2048, 16384, 1024),
                    make_sdesc_sw128(dO + k * 2048, 16384, 1024), IDESC_T, (it > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDK, make_sdesc_sw128(ds0 + k * 2048, 16384, 1024),
                    make_sdesc_sw128(q + k * 2048, 16384, 1024), IDESC_T, (it > 0 || k > 0));
        umma_commit(&empty[st]);
        umma_commit(pds_empty);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) { ok = issue_sdp(it + 1); if (!ok) break; }
        ok = issue_acc(it);
      }
      if (ok) umma_commit(acc_full);
      else { *abort_flag = ST_TIMEOUT_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else {
    // ------------------------------------------------------------ math warps
    const int quad = warp & 3, cb = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    const float dscale = dropout_scale(a.thr16);
    const long long bh = static_cast<long long>(b) * a.H + h;
    uint8_t* my_dq = sDQ + warp * 2048;
    bool ok = true;

    // drains dQ tile `it` (rows of query tile own+it, this warp's 16 columns) into the global
    // fp32 accumulator with one TMA reduce-add
    auto drain_dq = [&](int it) {
      if (!mbar_wait(&dq_full[it & 1], (it >> 1) & 1, abort_flag)) return false;
      tc_fence_after();
      uint32_t v[16];
      tmem_ld16(tDQ + (it & 1) * 64 + lane_addr + cb * 16, v);
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      tmem_ld_wait();
      tc_fence_before();
      // 16 fp32 columns = 64-byte rows, 64B swizzle
      uint8_t* rowp = my_dq + lane * 64;
      const int sw = (lane >> 1) & 3;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<float4*>(rowp + ((c ^ sw) << 4)) =
            make_float4(__uint_as_float(v[c * 4 + 0]), __uint_as_float(v[c * 4 + 1]),
                        __uint_as_float(v[c * 4 + 2]), __uint_as_float(v[c * 4 + 3]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&dq_empty[it & 1]);
        tma_reduce_add_2d(&tmDQ, my_dq, h * HD + cb * 16, b * a.T + (own + it) * 128 + quad * 32);
        tma_store_commit();
      }
      return true;
    };

    for (int it = 0; it < n_iter && ok; ++it) {
      const int qi = own + it;
      const int q_idx = qi * 128 + r;
      const bool q_ok = q_idx < a.T;
      const float lse_l2 = q_ok ? a.lse[bh * a.T + q_idx] * LOG2E : INFINITY;
      const float dlt = q_ok ? a.delta[bh * a.T + q_idx] : 0.f;
      const bool diag = it == 0;
      const uint64_t row_elem0 = (static_cast<uint64_t>(bh) * a.T + q_idx) * a.T + own * 128 + cb * 32;
      uint32_t keep32 = 0xffffffffu;
      if (a.thr16) {
        if (a.drop_mask) {
          keep32 = q_ok ? a.drop_mask[row_elem0 >> 5] : 0u;
        } else {
          keep32 = 0;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            keep32 |= dropout_keep8(salted(a.seed, a.salt), a.stream_id, (row_elem0 >> 3) + g, a.thr16) << (8 * g);
        }
      }
      if (!mbar_wait(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      if (it > 0 && !mbar_wait(pds_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int col0 = cb * 32 + hf * 16;
        uint32_t sv[16], dv[16];
        tmem_ld16(tS + lane_addr + col0, sv);
        tmem_ld16(tDP + lane_addr + col0, dv);
        tmem_ld_wait();
        float p[16], ds[16];
        const uint32_t k16 = keep32 >> (hf * 16);
        if (a.thr16) {
          if (diag) fb_math16<true, true>(sv, dv, p, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
          else      fb_math16<false, true>(sv, dv, p, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
        } else {
          if (diag) fb_math16<true, false>(sv, dv, p, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
          else      fb_math16<false, false>(sv, dv, p, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
        }
        const uint32_t poff = (col0 >> 6) * 16384;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t off = poff + sw128_chunk(r, ((col0 & 63) >> 3) + g);
          uint4 w;
          w.x = pack_bf16x2(p[g * 8 + 0], p[g * 8 + 1]); w.y = pack_bf16x2(p[g * 8 + 2], p[g * 8 + 3]);
          w.z = pack_bf16x2(p[g * 8 + 4], p[g * 8 + 5]); w.w = pack_bf16x2(p[g * 8 + 6], p[g * 8 + 7]);
          *reinterpret_cast<uint4*>(sP + off) = w;
          w.x = pack_bf16x2(ds[g * 8 + 0], ds[g * 8 + 1]); w.y = pack_bf16x2(ds[g * 8 + 2], ds[g * 8 + 3]);
          w.z = pack_bf16x2(ds[g * 8 + 4], ds[g * 8 + 5]); w.w = pack_bf16x2(ds[g * 8 + 6], ds[g * 8 + 7]);
          *reinterpret_cast<uint4*>(sDS + off) = w;
        }
      }
      // one arrival per warp: hundreds of threads arriving on one mbarrier serialise on it
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(sdp_empty); mbar_arrive(pds_full); }
      // the previous pair's dQ tile finished long ago: drain it while the tensor core works
      if (it > 0) ok = drain_dq(it - 1);
    }
    if (ok) ok = drain_dq(n_iter - 1);
    if (ok && !mbar_wait(acc_full, 0, abort_flag)) ok = false;
    if (!ok) { *abort_flag = ST_TIMEOUT_TMEM_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
    if (ok) {
      tc_fence_after();
      const int t_idx = own * 128 + r;
      __nv_bfloat16* base = a.dqkv + (static_cast<long long>(b) * a.T + t_idx) * (3 * d_model) + h * HD;
      // 4 chunks of 32 columns: dV chunks 0,1 then dK chunks 0,1; warp group cb takes chunk cb
      const uint32_t tacc = (cb < 2 ? tDV : tDK) + (cb & 1) * 32;
      __nv_bfloat16* dst = base + (cb < 2 ? 2 * d_model : d_model) + (cb & 1) * 32;
      uint32_t v[32];
      tmem_ld32(tacc + lane_addr, v);
      tmem_ld_wait();
      if (t_idx < a.T) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + q4 * 8) = w;
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == FB_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------
// Persistent form of the kernel above: one CTA per SM walks (batch*head) = blockIdx.x,
// blockIdx.x + gridDim.x, ... and, for each, the key tiles 0..nt-1, as ONE pipeline over
// (query tile, key tile) pairs.  K/V are double-buffered across key tiles, the Q/dO ring and the
// S/dP, P/dS and dQ hand-offs run on a pair counter that never restarts, and the end-of-tile work
// of key tile w (last dQ drain, dV/dK read-out and store) is done by the math warps after the
// P/dS math of the first pair of key tile w + 1, while the tensor core already works on that pair.
// So the per-key-tile prologue (TMEM allocation, barrier set-up, first loads) and tail, which cost
// as much as two pairs in the one-tile-per-CTA kernel, are paid once per CTA.

struct FbWalk {
  int bh, own, it, nt, bh_end, step;
  int w, g;      // key tiles and pairs done so far by this CTA
  __device__ __forceinline__ bool valid() const { return bh < bh_end; }
  __device__ __forceinline__ bool first() const { return it == 0; }
  __device__ __forceinline__ bool last() const { return it == nt - own - 1; }
  __device__ __forceinline__ void next() {
    ++g;
    if (++it == nt - own) {
      it = 0; ++w;
      if (++own == nt) { own = 0; bh += step; }
    }
  }
};

__global__ void __launch_bounds__(FB_THREADS, 1)
attn_bwd_fused64_persistent_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                   const __grid_constant__ CUtensorMap tmDO,
                                   const __grid_constant__ CUtensorMap tmDQ,
                                   const __grid_constant__ CUtensorMap tmDKV, const AttnBwdArgs a) {
  griddep_enter();
  constexpr int HD = 64;
  constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_T = make_idesc_bf16(128, HD, 1, 1);
  constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, HD, 0, 1);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sK = smem;                    // 2 stages
  uint8_t* sV = sK + 2 * FB_TILE;        // 2 stages
  uint8_t* sQ = sV + 2 * FB_TILE;        // 2 stages
  uint8_t* sDO = sQ + 2 * FB_TILE;       // 2 stages
  uint8_t* sP = sDO + 2 * FB_TILE;
  uint8_t* sDS = sP + FB_P;
  uint8_t* sDQ = sDS + FB_P;             // 16 warps x 2 KB staging for the dQ reduce-adds
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDQ + FB_MATH_WARPS * 2048);
  uint64_t* kv_full = bars;        // 2
  uint64_t* kv_empty = bars + 2;   // 2
  uint64_t* full = bars + 4;       // 2
  uint64_t* empty = bars + 6;      // 2
  uint64_t* sdp_full = bars + 8;
  uint64_t* sdp_empty = bars + 9;
  uint64_t* pds_full = bars + 10;
  uint64_t* pds_empty = bars + 11;
  uint64_t* dq_full = bars + 12;   // 2
  uint64_t* dq_empty = bars + 14;  // 2
  uint64_t* acc_full = bars + 16;
  uint64_t* acc_empty = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (a.T + 127) / 128;
  const int d_model = a.H * HD;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&full[i], 1); mbar_init(&empty[i], 1);
      mbar_init(&dq_full[i], 1); mbar_init(&dq_empty[i], FB_MATH_WARPS);
    }
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, FB_MATH_WARPS);
    mbar_init(pds_full, FB_MATH_WARPS); mbar_init(pds_empty, 1);
    mbar_init(acc_full, 1); mbar_init(acc_empty, FB_MATH_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
    tma_prefetch_desc(&tmDKV);
  }
  if (warp == FB_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 320,
                 tDQ = tmem_base + 384;
  FbWalk start;
  start.bh = static_cast<int>(blockIdx.x); start.own = 0; start.it = 0; start.nt = nt;
  start.bh_end = a.B * a.H; start.step = static_cast<int>(gridDim.x); start.w = 0; start.g = 0;

  if (warp == FB_TMA_WARP) {
    if (lane == 0) {
      for (FbWalk p = start; p.valid(); p.next()) {
        const int b = p.bh / a.H, h = p.bh % a.H;
        if (p.first()) {
          const int s = p.w & 1;
          if (!mbar_wait(&kv_empty[s], ((p.w >> 1) & 1) ^ 1, abort_flag)) {
            *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break;
          }
          const int row_own = b * a.T + p.own * 128;
          mbar_expect_tx(&kv_full[s], 2 * FB_TILE);
          tma_load_2d(sK + s * FB_TILE, &tmQKV, &kv_full[s], d_model + h * HD, row_own);
          tma_load_2d(sV + s * FB_TILE, &tmQKV, &kv_full[s], 2 * d_model + h * HD, row_own);
        }
        const int st = p.g & 1;
        const int row = b * a.T + (p.own + p.it) * 128;
        if (!mbar_wait(&empty[st], ((p.g >> 1) & 1) ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break;
        }
        mbar_expect_tx(&full[st], 2 * FB_TILE);
        tma_load_2d(sQ + st * FB_TILE, &tmQKV, &full[st], h * HD, row);
        tma_load_2d(sDO + st * FB_TILE, &tmDO, &full[st], h * HD, row);
      }
    }
  } else if (warp == FB_MMA_WARP) {
    if (lane == 0) {
      const uint32_t p0 = smem_u32(sP), ds0 = smem_u32(sDS);
      auto issue_sdp = [&](const FbWalk& p) {
        const int st = p.g & 1;
        if (p.first() && !mbar_wait(&kv_full[p.w & 1], (p.w >> 1) & 1, abort_flag)) return false;
        if (!mbar_wait(&full[st], (p.g >> 1) & 1, abort_flag)) return false;
        if (p.g > 0 && !mbar_wait(sdp_empty, (p.g - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k0 = smem_u32(sK + (p.w & 1) * FB_TILE), v0 = smem_u32(sV + (p.w & 1) * FB_TILE);
        const uint32_t q = smem_u32(sQ + st * FB_TILE), dO = smem_u32(sDO + st * FB_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tS, make_sdesc_sw128(q + k * 32, 16, 1024), make_sdesc_sw128(k0 + k * 32, 16, 1024),
                    IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tDP, make_sdesc_sw128(dO + k * 32, 16, 1024), make_sdesc_sw128(v0 + k * 32, 16, 1024),
                    IDESC_S, k > 0);
        umma_commit(sdp_full);
        return true;
      };
      auto issue_acc = [&](const FbWalk& p) {
        const int st = p.g & 1;
        if (!mbar_wait(pds_full, p.g & 1, abort_flag)) return false;
        if (p.g >= 2 && !mbar_wait(&dq_empty[p.g & 1], ((p.g - 2) >> 1) & 1, abort_flag)) return false;
        // dV / dK of the previous key tile must have been read out before they are overwritten
        if (p.first() && p.w > 0 && !mbar_wait(acc_empty, (p.w - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k0 = smem_u32(sK + (p.w & 1) * FB_TILE);
        const uint32_t q = smem_u32(sQ + st * FB_TILE), dO = smem_u32(sDO + st * FB_TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDQ + (p.g & 1) * 64, make_sdesc_sw128(ds0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                    make_sdesc_sw128(k0 + k * 2048, 16384, 1024), IDESC_DQ, k > 0);
        umma_commit(&dq_full[p.g & 1]);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDV, make_sdesc_sw128(p0 + k * 2048, 16384, 1024),
                    make_sdesc_sw128(dO + k * 2048, 16384, 1024), IDESC_T, (p.it > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tDK, make_sdesc_sw128(ds0 + k * 2048, 16384, 1024),
                    make_sdesc_sw128(q + k * 2048, 16384, 1024), IDESC_T, (p.it > 0 || k > 0));
        umma_commit(&empty[st]);
        umma_commit(pds_empty);
        if (p.last()) {
          umma_commit(acc_full);                 // dV / dK of this key tile complete
          umma_commit(&kv_empty[p.w & 1]);       // and its K / V stage is free
        }
        return true;
      };
      FbWalk cur = start, nxt = start;
      bool ok = true;
      if (cur.valid()) { nxt.next(); ok = issue_sdp(cur); }
      while (ok && cur.valid()) {
        if (nxt.valid()) { ok = issue_sdp(nxt); if (!ok) break; }
        ok = issue_acc(cur);
        cur = nxt;
        if (nxt.valid()) nxt.next();
      }
      if (!ok) { *abort_flag = ST_TIMEOUT_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else {
    // ------------------------------------------------------------ math warps
    const int quad = warp & 3, cb = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    const float dscale = dropout_scale(a.thr16);
    uint8_t* my_dq = sDQ + warp * 2048;
    bool ok = true;

    // drains the dQ tile of pair g (query rows starting at global row `row0` of head h, this
    // warp's 16 columns) into the global fp32 accumulator with one TMA reduce-add
    auto drain_dq = [&](int g, int row0, int h) {
      if (!mbar_wait(&dq_full[g & 1], (g >> 1) & 1, abort_flag)) return false;
      tc_fence_after();
      uint32_t v[16];
      tmem_ld16(tDQ + (g & 1) * 64 + lane_addr + cb * 16, v);
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      tmem_ld_wait();
      tc_fence_before();
      uint8_t* rowp = my_dq + lane * 64;       // 16 fp32 columns = 64-byte rows, 64B swizzle
      const int sw = (lane >> 1) & 3;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<float4*>(rowp + ((c ^ sw) << 4)) =
            make_float4(__uint_as_float(v[c * 4 + 0]), __uint_as_float(v[c * 4 + 1]),
                        __uint_as_float(v[c * 4 + 2]), __uint_as_float(v[c * 4 + 3]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&dq_empty[g & 1]);
        tma_reduce_add_2d(&tmDQ, my_dq, h * HD + cb * 16, row0 + quad * 32);
        tma_store_commit();
      }
      return true;
    };
    // reads the finished dV / dK of key tile w out of TMEM, frees them, and stores them
    auto finish_tile = [&](int w, int b, int h, int own) {
      if (!mbar_wait(acc_full, w & 1, abort_flag)) return false;
      tc_fence_after();
      // 4 chunks of 32 columns: dV chunks 0,1 then dK chunks 0,1; warp group cb takes chunk cb
      const uint32_t tacc = (cb < 2 ? tDV : tDK) + (cb & 1) * 32;
      uint32_t v[32];
      tmem_ld32(tacc + lane_addr, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      if ((a.T & 127) == 0) {
        // 32 rows x 32 bf16 columns per warp: staged with 64-byte swizzle, one TMA store.  (Plain
        // stores of 64-byte row pieces 6 KB apart kept the load/store unit busy for thousands of
        // cycles per key tile and delayed every other warp's shared-memory traffic with them.)
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        uint8_t* rowp = my_dq + lane * 64;
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 wv;
          wv.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
          wv.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
          wv.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
          wv.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
          *reinterpret_cast<uint4*>(rowp + ((q4 ^ sw) << 4)) = wv;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmDKV, my_dq, (cb < 2 ? 2 * d_model : d_model) + h * HD + (cb & 1) * 32,
                       b * a.T + own * 128 + quad * 32);
          tma_store_commit();
        }
        return true;
      }
      // ragged last tile: rows past T belong to the next sequence, so store row by row
      const int t_idx = own * 128 + r;
      if (t_idx < a.T) {
        __nv_bfloat16* dst = a.dqkv + (static_cast<long long>(b) * a.T + t_idx) * (3 * d_model) + h * HD +
                             (cb < 2 ? 2 * d_model : d_model) + (cb & 1) * 32;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 wv;
          wv.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
          wv.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
          wv.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
          wv.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + q4 * 8) = wv;
        }
      }
      return true;
    };

    int prev_row0 = 0, prev_h = 0, prev_b = 0, prev_own = 0;     // pair g - 1 / its key tile
    // per-row inputs of a pair: log-sum-exp, delta and the 32 dropout keep bits of this thread's
    // columns.  They are fetched one pair ahead so their latency never sits in the pair's chain.
    // Addresses advance by fixed strides from one query tile to the next, so they are rebuilt from
    // the indices only at the first pair of a key tile.
    long long row_off = 0;          // (batch*head) * T + query index of this thread's row
    long long keep_off = 0;         // word index of its 32 keep bits
    // (fetch only issues the loads: no arithmetic on the loaded values here, so nothing waits for
    // them before the next pair needs them)
    auto fetch = [&](const FbWalk& w, float& lse_raw, float& dlt, uint32_t& keep32) {
      const int q_idx = (w.own + w.it) * 128 + r;
      const bool q_ok = q_idx < a.T;
      if (w.it == 0) {
        row_off = static_cast<long long>(w.bh) * a.T + q_idx;
        keep_off = (row_off * a.T + w.own * 128 + cb * 32) >> 5;
      } else {
        row_off += 128;
        keep_off += 4ll * a.T;      // 128 rows of T / 32 words
      }
      lse_raw = INFINITY;
      dlt = 0.f;
      if (q_ok) { lse_raw = a.lse[row_off]; dlt = a.delta[row_off]; }
      keep32 = 0xffffffffu;
      if (a.thr16) {
        if (a.drop_mask) {
          keep32 = 0u;
          if (q_ok) keep32 = a.drop_mask[keep_off];
        } else {
          const uint64_t row_elem0 = static_cast<uint64_t>(row_off) * a.T + w.own * 128 + cb * 32;
          keep32 = 0;
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4)
            keep32 |= dropout_keep8(salted(a.seed, a.salt), a.stream_id, (row_elem0 >> 3) + g4, a.thr16) << (8 * g4);
        }
      }
    };
    FbWalk p = start;
    int b = 0, h = 0;
    float lse_raw = 0.f, dlt = 0.f;
    uint32_t keep32 = 0xffffffffu;
    if (p.valid()) fetch(p, lse_raw, dlt, keep32);
    for (; p.valid() && ok; p.next()) {
      if (p.it == 0 && p.own == 0) { b = p.bh / a.H; h = p.bh - b * a.H; }
      const int qi = p.own + p.it;
      const int q_idx = qi * 128 + r;
      const bool q_ok = q_idx < a.T;
      const bool diag = p.it == 0;
      float n_lse = 0.f, n_dlt = 0.f;
      uint32_t n_keep = 0xffffffffu;
      {
        FbWalk q = p;
        q.next();
        if (q.valid()) fetch(q, n_lse, n_dlt, n_keep);
      }
      if (!mbar_wait(sdp_full, p.g & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float lse_l2 = lse_raw * LOG2E;          // +inf for rows outside the sequence
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int col0 = cb * 32 + hf * 16;
        uint32_t sv[16], dv[16];
        tmem_ld16(tS + lane_addr + col0, sv);
        tmem_ld16(tDP + lane_addr + col0, dv);
        tmem_ld_wait();
        float pp[16], ds[16];
        const uint32_t k16 = keep32 >> (hf * 16);
        if (a.thr16) {
          if (diag) fb_math16<true, true>(sv, dv, pp, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
          else      fb_math16<false, true>(sv, dv, pp, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
        } else {
          if (diag) fb_math16<true, false>(sv, dv, pp, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
          else      fb_math16<false, false>(sv, dv, pp, ds, r, col0, sl2, lse_l2, dlt * a.scale, a.scale, dscale, k16);
        }
        if (hf == 0) {
          // the shared P / dS tiles feed the previous pair's dV / dK / dQ products until
          // pds_empty completes; the first half of this pair's math has run under them
          if (p.g > 0 && !mbar_wait(pds_empty, (p.g - 1) & 1, abort_flag)) { ok = false; break; }
        }
        const uint32_t poff = (col0 >> 6) * 16384;
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
          const uint32_t off = poff + sw128_chunk(r, ((col0 & 63) >> 3) + g2);
          uint4 wv;
          wv.x = pack_bf16x2(pp[g2 * 8 + 0], pp[g2 * 8 + 1]); wv.y = pack_bf16x2(pp[g2 * 8 + 2], pp[g2 * 8 + 3]);
          wv.z = pack_bf16x2(pp[g2 * 8 + 4], pp[g2 * 8 + 5]); wv.w = pack_bf16x2(pp[g2 * 8 + 6], pp[g2 * 8 + 7]);
          *reinterpret_cast<uint4*>(sP + off) = wv;
          wv.x = pack_bf16x2(ds[g2 * 8 + 0], ds[g2 * 8 + 1]); wv.y = pack_bf16x2(ds[g2 * 8 + 2], ds[g2 * 8 + 3]);
          wv.z = pack_bf16x2(ds[g2 * 8 + 4], ds[g2 * 8 + 5]); wv.w = pack_bf16x2(ds[g2 * 8 + 6], ds[g2 * 8 + 7]);
          *reinterpret_cast<uint4*>(sDS + off) = wv;
        }
      }
      if (!ok) break;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(sdp_empty); mbar_arrive(pds_full); }
      // work left over from the previous pair, done while the tensor core runs this one
      if (p.g > 0) {
        ok = drain_dq(p.g - 1, prev_row0, prev_h);
        if (ok && p.first()) ok = finish_tile(p.w - 1, prev_b, prev_h, prev_own);
      }
      prev_row0 = b * a.T + qi * 128; prev_h = h; prev_b = b; prev_own = p.own;
      lse_raw = n_lse; dlt = n_dlt; keep32 = n_keep;
    }
    if (ok && p.g > 0) {
      ok = drain_dq(p.g - 1, prev_row0, prev_h);
      if (ok) ok = finish_tile(p.w - 1, prev_b, prev_h, prev_own);
    }
    if (!ok) { *abort_flag = ST_TIMEOUT_TMEM_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
    if (lane == 0) tma_store_wait<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == FB_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}


// dqkv[:, 0:d] = bf16(dq_acc).  A block walks whole rows (thread = one float4 column group), so
// every access is a contiguous row segment.  The accumulator is cleared by a separate memset:
// overwriting each element right after loading it in the same kernel measured ten times slower
// on B200 than the read-only conversion plus a memset.
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, int rows, int d) {
  griddep_enter();
  const int d4 = d >> 2;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* src = reinterpret_cast<const float4*>(acc + static_cast<long long>(row) * d);
    uint2* dst = reinterpret_cast<uint2*>(dqkv + static_cast<long long>(row) * 3 * d);
    for (int c4 = threadIdx.x; c4 < d4; c4 += 256) {
      const float4 v = src[c4];
      uint2 o;
      o.x = pack_bf16x2(v.x, v.y);
      o.y = pack_bf16x2(v.z, v.w);
      dst[c4] = o;
    }
  }
}

// 0 = choose by problem shape, 1 = one key tile per CTA, 2 = persistent walk
static int g_attn_bwd_schedule = -1;
static int attn_bwd_schedule_mode() {
  if (g_attn_bwd_schedule < 0) {
    const char* v = getenv("AB_ATTN_BWD_SCHEDULE");
    g_attn_bwd_schedule = (v && v[0] >= '0' && v[0] <= '2') ? v[0] - '0' : 0;
  }
  return g_attn_bwd_schedule;
}

int launch_attn_bwd_fused64(const CUtensorMap& tq, const CUtensorMap& td, const AttnBwdArgs& a,
                            cudaStream_t stream) {
  CUtensorMap tdq;
  const long long rows = static_cast<long long>(a.B) * a.T;
  const int d = a.H * 64;
  int rc = make_tmap_2d_sw(&tdq, a.dq_acc, rows, d, d, 32, 16, 4, 64);
  if (rc) return rc;
  // the persistent walk hands whole (batch, head) slices to CTAs, which only balances with several
  // slices per SM; few, long slices go to the one-tile-per-CTA grid
  const int mode = attn_bwd_schedule_mode();
  if (mode == 1 || (mode == 0 && a.B * a.H < 4 * 148)) {
    constexpr int SMEM = 6 * FB_TILE + 2 * FB_P + FB_MATH_WARPS * 2048 + 256;
    static PerDeviceOnce attr;
    if (attr.first_use_on_device()) {
      cudaError_t e = cudaFuncSetAttribute(attn_bwd_fused64_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
      if (e != cudaSuccess) return (int)e;
      attr.mark_device();
    }
    dim3 grid((a.T + 127) / 128, a.H, a.B);
    launch_chained(attn_bwd_fused64_kernel, dim3(grid), dim3(FB_THREADS), SMEM, stream, tq, td, tdq, a);
  } else {
    constexpr int SMEM = 8 * FB_TILE + 2 * FB_P + FB_MATH_WARPS * 2048 + 256;
    static PerDeviceOnce attr;
    if (attr.first_use_on_device()) {
      cudaError_t e = cudaFuncSetAttribute(attn_bwd_fused64_persistent_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
      if (e != cudaSuccess) return (int)e;
      attr.mark_device();
    }
    CUtensorMap tdkv;     // the packed dQKV activation, boxes of 32 rows x 32 columns for dK / dV
    rc = make_tmap_2d_sw(&tdkv, a.dqkv, rows, 3 * d, 3 * d, 32, 32, 2, 64);
    if (rc) return rc;
    const int bh = a.B * a.H;
    launch_chained(attn_bwd_fused64_persistent_kernel, dim3(bh < 148 ? bh : 148), dim3(FB_THREADS), SMEM, stream, tq, td, tdq,
                                                                                          tdkv, a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  launch_chained(attn_dq_convert_kernel, dim3(148 * 16), dim3(256), 0, stream, a.dq_acc, a.dqkv, (int)rows, d);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemsetAsync(a.dq_acc, 0, sizeof(float) * rows * d, stream);
}

}  // namespace ab

// Schedule of the head_dim-64 backward: 0 = by problem shape (default; also read once from the
// environment variable AB_ATTN_BWD_SCHEDULE), 1 = one key tile per CTA, 2 = persistent walk.
extern "C" int ab_attn_bwd_schedule(int mode) {
  if (mode < 0 || mode > 2) return -1;
  ab::g_attn_bwd_schedule = mode;
  return 0;
}

// Stand-alone entry to the dQ conversion (bf16 copy into the packed dQKV activation, then clear).
extern "C" int ab_attn_dq_convert(float* acc, void* dqkv, int rows, int d, cudaStream_t stream) {
  ab::launch_chained(ab::attn_dq_convert_kernel, dim3(148 * 16), dim3(256), 0, stream, acc, (__nv_bfloat16*)dqkv, rows, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)rows * d, stream);
}
