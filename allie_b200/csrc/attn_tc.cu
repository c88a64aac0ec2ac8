// Causal flash attention on tcgen05 (forward; the backward kernels follow further down).
//
// One CTA owns one 128-row query tile of one (batch, head).  Per 128-row key/value tile:
//   warp 5 (one thread) : S = Q K^T          -> TMEM (128 lanes = query rows, 128 fp32 columns)
//   warps 0-3           : tcgen05.ld S, online softmax (row = thread), dropout, P -> smem (bf16,
//                         128B-swizzled panels = the UMMA K-major A layout)
//   warp 5              : PV = P V           -> TMEM (fresh, not accumulated)
//   warps 0-3           : O = O * alpha + PV in registers
//   warp 4 (one thread) : TMA loads of Q once and K/V tiles through a 2-stage ring
// Q, K and V are read straight out of the packed [B*T, 3*d] QKV activation with 2-D TMA boxes
// (64 columns x 128 rows), and O is written in the [B*T, d] layout the projection GEMM reads.
// V is consumed MN-major (rows = keys), so no transposes exist anywhere.
#include "attn_common.cuh"

namespace ab {

constexpr int FWD_MATH_WARPS = 8;
constexpr int FWD_MATH_THREADS = FWD_MATH_WARPS * 32;
constexpr int FWD_TMA_WARP = FWD_MATH_WARPS;
constexpr int FWD_MMA_WARP = FWD_MATH_WARPS + 1;
constexpr int FWD_THREADS = (FWD_MATH_WARPS + 2) * 32;

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, HD <= 64 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmO,
                const AttnArgs a) {
  griddep_enter();
  constexpr int PANELS = HD / 64;               // 64-column panels per Q/K/V tile
  constexpr int TILE_BYTES = 128 * HD * 2;      // one Q / K / V tile
  constexpr int P_BYTES = 128 * 128 * 2;
  constexpr int TMEM_COLS = (128 + HD) <= 256 ? 256 : 512;
  constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(128, HD, 0, 1);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;        // 2 stages
  uint8_t* sP = sV + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // 2
  uint64_t* v_full = bars + 3;              // 2
  uint64_t* k_empty = bars + 5;             // 2
  uint64_t* v_empty = bars + 7;             // 2
  uint64_t* s_full = bars + 9;
  uint64_t* s_empty = bars + 10;
  uint64_t* p_full = bars + 11;
  uint64_t* pv_full = bars + 12;
  uint64_t* pv_empty = bars + 13;
  // row statistics exchange between the two column halves: one barrier per TMEM lane quarter,
  // shared by the two warps that own the same 32 query rows (the quarters do not wait for each other)
  uint64_t* xchg = bars + 14 + (threadIdx.x >> 5 & 3);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_stat = reinterpret_cast<int*>(tmem_slot + 2);       // [128 rows] running row maximum (ordered-int coded)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (a.T + AT_BM - 1) / AT_BM;
  const int qt = nqt - 1 - blockIdx.x;      // heaviest tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int nkv = qt + 1;                   // causal: key tiles 0..qt
  const int d_model = a.H * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1); mbar_init(s_empty, FWD_MATH_WARPS);
    mbar_init(p_full, FWD_MATH_WARPS); mbar_init(pv_full, 1); mbar_init(pv_empty, FWD_MATH_WARPS);
    for (int i = 0; i < 4; ++i) mbar_init(bars + 14 + i, 2);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
  }
  if (threadIdx.x < 128) s_stat[threadIdx.x] = ord_encode(-INFINITY);
  if (warp == FWD_MMA_WARP) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tPV = tmem_base + 128;

  if (warp == FWD_TMA_WARP) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int row_q = b * a.T + qt * AT_BM;
      mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int p = 0; p < PANELS; ++p)
        tma_load_2d(sQ + p * 16384, &tmQKV, q_full, h * HD + p * 64, row_q);
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        const int row_k = b * a.T + j * AT_BN;
        if (!mbar_wait(&k_empty[st], par, abort_flag)) { *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          tma_load_2d(sK + st * TILE_BYTES + p * 16384, &tmQKV, &k_full[st],
                      d_model + h * HD + p * 64, row_k);
        if (!mbar_wait(&v_empty[st], par, abort_flag)) { *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          tma_load_2d(sV + st * TILE_BYTES + p * 16384, &tmQKV, &v_full[st],
                      2 * d_model + h * HD + p * 64, row_k);
      }
    }
  } else if (warp == FWD_MMA_WARP) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, abort_flag)) return false;
        if (j > 0 && !mbar_wait(s_empty, (j - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q0 = smem_u32(sQ), k0 = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16(tS, make_sdesc_sw128(q0 + off, 16, 1024), make_sdesc_sw128(k0 + off, 16, 1024),
                    IDESC_S, k > 0);
        }
        umma_commit(&k_empty[st]);
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < nkv) { ok = issue_qk(j + 1); if (!ok) break; }
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
        if (j > 0 && !mbar_wait(pv_empty, (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p0 = smem_u32(sP), v0 = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 128 keys = 8 UMMA_K steps
          const uint64_t adesc = make_sdesc_sw128(p0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_sdesc_sw128(v0 + k * 2048, 16384, 1024);
          umma_bf16(tPV, adesc, bdesc, IDESC_PV, k > 0);
        }
        umma_commit(&v_empty[st]);
        umma_commit(pv_full);
      }
      if (!ok) { *abort_flag = ST_TIMEOUT_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else {
    // ---------------------------------------------------- softmax / output warps
    // warp w: TMEM lane quarter w & 3 (query rows), column half w >> 2 (64 keys of each tile and
    // HD/2 output columns).  The halves exchange their partial row maxima through shared memory.
    const int r = (warp & 3) * 32 + lane;         // query row inside the tile = TMEM lane
    const int hf = warp >> 2;
    const int q_idx = qt * AT_BM + r;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    constexpr int OC = HD / 2;                    // output columns owned by this thread
    float m_run = -INFINITY, l_part = 0.f;
    float o[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o[i] = 0.f;
    const float dscale = dropout_scale(a.thr16);
    const uint64_t row_elem0 = (static_cast<uint64_t>(b * a.H + h) * a.T + q_idx) * a.T + hf * 64;
    bool ok = true;
    // Dropout keep bits of this thread's 64 keys of one key tile (two words of 32).  They do not
    // depend on the scores, so the generator runs for tile j + 1 while the tensor core computes
    // P V of tile j (the math warps would only be waiting then); the words are also what the
    // backward pass reads back, so it never re-runs the generator.
    uint32_t keep_w0 = 0xffffffffu, keep_w1 = 0xffffffffu;
    auto make_keep = [&](int j) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint64_t e0 = row_elem0 + static_cast<uint64_t>(j) * AT_BN + c * 32;
        uint32_t word = 0;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          word |= dropout_keep8(salted(a.seed, a.salt), a.stream_id, (e0 >> 3) + g, a.thr16) << (8 * g);
        if (c == 0) keep_w0 = word; else keep_w1 = word;
        if (a.drop_mask && q_idx < a.T) a.drop_mask[e0 >> 5] = word;
      }
    };
    if (a.thr16 && nkv > 0) make_keep(0);
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qt);
      // pass 1: partial row maximum over this half's 64 keys
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tS + lane_addr + hf * 64 + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sc = __uint_as_float(v[i]);
          if (!diag || (hf * 64 + c * 32 + i) <= r) mx = fmaxf(mx, sc);
        }
      }
      // running maximum of the row, shared by the two column halves (monotone, so one slot per
      // row updated with atomicMax is enough; its last reader is ordered before its next writer by
      // the s_empty -> next S chain)
      atomicMax(&s_stat[r], ord_encode(mx));
      __syncwarp();
      if (lane == 0) mbar_arrive(xchg);     // one arrival per warp (see below)
      if (!mbar_wait(xchg, j & 1, abort_flag)) { ok = false; break; }
      const float m_new = ord_decode(s_stat[r]);   // finite: key 0 is never masked
      const float alpha = ex2_fast((m_run - m_new) * sl2);
      const float mb = m_new * sl2;
      float rs = 0.f;
      // pass 2: probabilities -> smem (bf16), partial row sum
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tS + lane_addr + hf * 64 + c * 32, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = ex2_fast(__uint_as_float(v[i]) * sl2 - mb);
          p[i] = (!diag || (hf * 64 + c * 32 + i) <= r) ? e : 0.f;
          rs += p[i];
        }
        if (a.thr16) {
          const uint32_t word = c ? keep_w1 : keep_w0;
#pragma unroll
          for (int i = 0; i < 32; ++i) p[i] = ((word >> i) & 1u) ? p[i] * dscale : 0.f;
        }
        uint8_t* panel = sP + hf * 16384;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16x2(p[g * 8 + 0], p[g * 8 + 1]); w.y = pack_bf16x2(p[g * 8 + 2], p[g * 8 + 3]);
          w.z = pack_bf16x2(p[g * 8 + 4], p[g * 8 + 5]); w.w = pack_bf16x2(p[g * 8 + 6], p[g * 8 + 7]);
          *reinterpret_cast<uint4*>(panel + sw128_chunk(r, c * 4 + g)) = w;
        }
      }
      // one arrival per warp: hundreds of threads arriving on one mbarrier serialise on it
      tc_fence_before();
      fence_proxy_async_smem();          // P visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) { mbar_arrive(s_empty); mbar_arrive(p_full); }   // S reusable, P ready
      l_part = l_part * alpha + rs;
      m_run = m_new;
      if (a.thr16 && j + 1 < nkv) make_keep(j + 1);
      // fold in this tile's PV (this thread's HD/2 output columns)
      if (!mbar_wait(pv_full, j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tPV + lane_addr + hf * OC + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_empty);
    }
    // total row sum = sum of the two halves' partial sums: half 1 publishes its part, half 0 adds
    // its own and publishes the total (two rounds through the same slot)
    if (ok) {
      float* fs = reinterpret_cast<float*>(s_stat);
      if (hf == 1) fs[r] = l_part;
      __syncwarp();
      if (lane == 0) mbar_arrive(xchg);
      if (!mbar_wait(xchg, nkv & 1, abort_flag)) ok = false;
      if (ok && hf == 0) { l_part += fs[r]; fs[r] = l_part; }
      __syncwarp();
      if (lane == 0) mbar_arrive(xchg);
      if (ok && !mbar_wait(xchg, (nkv + 1) & 1, abort_flag)) ok = false;
      if (ok && hf == 1) l_part = fs[r];
    }
    if (!ok) { *abort_flag = ST_TIMEOUT_TMEM_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
    if (ok && (a.T & 127) == 0) {
      // Whole tile in range: the warp stages its 32 rows x HD/2 columns in the (now idle) P tile
      // and stores them with one TMA store.  Direct stores of 64-byte row pieces one row pitch
      // apart keep the load/store unit busy far longer than the bytes justify.
      const float inv = 1.f / l_part;
      constexpr int ROW_BYTES = OC * 2;                 // 64 (64B swizzle) or 128 (128B swizzle)
      uint8_t* stg = sP + warp * (32 * ROW_BYTES);
      uint8_t* rowp = stg + lane * ROW_BYTES;
      const int sw = ROW_BYTES == 64 ? ((lane >> 1) & 3) : (lane & 7);
#pragma unroll
      for (int g = 0; g < OC / 8; ++g) {
        uint4 w;
        w.x = pack_bf16x2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv);
        w.y = pack_bf16x2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
        w.z = pack_bf16x2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv);
        w.w = pack_bf16x2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(rowp + ((g ^ sw) << 4)) = w;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmO, stg, h * HD + hf * OC, b * a.T + qt * AT_BM + (warp & 3) * 32);
        tma_store_commit();
      }
      if (a.lse && hf == 0) a.lse[(static_cast<long long>(b) * a.H + h) * a.T + q_idx] = m_run * a.scale + logf(l_part);
      if (lane == 0) tma_store_wait_read<0>();          // the staging tile outlives the read
    } else if (ok && q_idx < a.T) {
      const float inv = 1.f / l_part;
      __nv_bfloat16* orow = a.out + (static_cast<long long>(b) * a.T + q_idx) * d_model + h * HD + hf * OC;
#pragma unroll
      for (int g = 0; g < OC / 8; ++g) {
        uint4 w;
        w.x = pack_bf16x2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv);
        w.y = pack_bf16x2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
        w.z = pack_bf16x2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv);
        w.w = pack_bf16x2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(orow + g * 8) = w;
      }
      if (a.lse && hf == 0) a.lse[(static_cast<long long>(b) * a.H + h) * a.T + q_idx] = m_run * a.scale + logf(l_part);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == FWD_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace ab

// =================================================================================================
// Backward.  Two launches of one templated kernel, both with threads = query rows:
//   MODE 0 (key/value-stationary): CTA owns key tile j, streams query tiles i >= j, accumulates
//           dV_j += P^T dO_i and dK_j += dS^T Q_i in TMEM.
//   MODE 1 (query-stationary)    : CTA owns query tile i, streams key tiles j <= i, accumulates
//           dQ_i += dS K_j in TMEM.
// Both recompute S = Q K^T and dP = dO V^T per tile pair, so no atomics and no fp32 dQ buffer
// are needed.  P and dS are written once to shared memory as [query row][key] bf16 panels; that
// one layout is the K-major A operand of dS*K and the MN-major A operand of P^T*dO / dS^T*Q.
// delta[b,h,t] = sum_c dO*O is produced by a small pre-kernel.
namespace ab {


// One thread per 16-byte chunk of O / dO (hd / 8 adjacent lanes share one (row, head)), so a
// warp reads 512 contiguous bytes of each tensor; the lanes of a (row, head) fold their partial
// dot products with shuffles.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                  float* __restrict__ delta, int B, int T, int H, int hd) {
  griddep_enter();
  const int cpr = hd >> 3;                                    // chunks per (row, head): 8 or 16
  const long long total = static_cast<long long>(B) * T * H * cpr;
  const long long gid = blockIdx.x * 256ll + threadIdx.x;
  float s = 0.f;
  if (gid < total) {
    const uint4 x = __ldcs(reinterpret_cast<const uint4*>(o) + gid);
    const uint4 y = __ldcs(reinterpret_cast<const uint4*>(dout) + gid);
    s = bf16_lo(x.x) * bf16_lo(y.x) + bf16_hi(x.x) * bf16_hi(y.x);
    s += bf16_lo(x.y) * bf16_lo(y.y) + bf16_hi(x.y) * bf16_hi(y.y);
    s += bf16_lo(x.z) * bf16_lo(y.z) + bf16_hi(x.z) * bf16_hi(y.z);
    s += bf16_lo(x.w) * bf16_lo(y.w) + bf16_hi(x.w) * bf16_hi(y.w);
  }
  for (int off = 1; off < cpr; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (gid < total && (gid & (cpr - 1)) == 0) {
    const long long rh = gid / cpr;                           // row * H + head
    const int hh = static_cast<int>(rh % H);
    const long long row = rh / H;
    const int bb = static_cast<int>(row / T), t = static_cast<int>(row % T);
    delta[(static_cast<long long>(bb) * H + hh) * T + t] = s;
  }
}

constexpr int BWD_MATH_WARPS = 16;
constexpr int BWD_MATH_THREADS = BWD_MATH_WARPS * 32;
constexpr int BWD_TMA_WARP = BWD_MATH_WARPS;
constexpr int BWD_MMA_WARP = BWD_MATH_WARPS + 1;
constexpr int BWD_THREADS = (BWD_MATH_WARPS + 2) * 32;

template <int HD, int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                const AttnBwdArgs a) {
  griddep_enter();
  constexpr int STAGES = HD <= 64 ? 2 : 1;
  constexpr int PANELS = HD / 64;
  constexpr int TILE_BYTES = 128 * HD * 2;
  constexpr int P_BYTES = 128 * 128 * 2;
  constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);     // Q K^T and dO V^T
  constexpr uint32_t IDESC_T = make_idesc_bf16(128, HD, 1, 1);      // P^T dO, dS^T Q (both MN-major)
  constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, HD, 0, 1);     // dS K

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sStatA = smem;                                  // MODE 0: K_j   MODE 1: Q_i
  uint8_t* sStatB = sStatA + TILE_BYTES;                   // MODE 0: V_j   MODE 1: dO_i
  uint8_t* sStrX = sStatB + TILE_BYTES;                    // MODE 0: Q_i   MODE 1: K_j   (STAGES)
  uint8_t* sStrY = sStrX + STAGES * TILE_BYTES;            // MODE 0: dO_i  MODE 1: V_j   (STAGES)
  uint8_t* sP = sStrY + STAGES * TILE_BYTES;
  uint8_t* sDS = sP + P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + P_BYTES);
  uint64_t* stat_full = bars;
  uint64_t* full = bars + 1;        // STAGES
  uint64_t* empty = bars + 3;       // STAGES
  uint64_t* sdp_full = bars + 5;
  uint64_t* sdp_empty = bars + 6;
  uint64_t* pds_full = bars + 7;
  uint64_t* pds_empty = bars + 8;
  uint64_t* acc_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (a.T + 127) / 128;
  const int h = blockIdx.y, b = blockIdx.z;
  // MODE 0: own key tile `own`, iterate query tiles own..nt-1 (heaviest = small own first)
  // MODE 1: own query tile `own`, iterate key tiles 0..own (heaviest = large own first)
  const int own = MODE == 0 ? static_cast<int>(blockIdx.x) : nt - 1 - static_cast<int>(blockIdx.x);
  const int n_iter = MODE == 0 ? nt - own : own + 1;
  const int d_model = a.H * HD;

  if (threadIdx.x == 0) {
    mbar_init(stat_full, 1);
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, BWD_MATH_WARPS);
    mbar_init(pds_full, BWD_MATH_WARPS); mbar_init(pds_empty, 1); mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == BWD_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tAcc0 = tmem_base + 256,
                 tAcc1 = tmem_base + 256 + HD;

  if (warp == BWD_TMA_WARP) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int row_own = b * a.T + own * 128;
      mbar_expect_tx(stat_full, 2 * TILE_BYTES);
#pragma unroll
      for (int p = 0; p < PANELS; ++p) {
        if (MODE == 0) {
          tma_load_2d(sStatA + p * 16384, &tmQKV, stat_full, d_model + h * HD + p * 64, row_own);
          tma_load_2d(sStatB + p * 16384, &tmQKV, stat_full, 2 * d_model + h * HD + p * 64, row_own);
        } else {
          tma_load_2d(sStatA + p * 16384, &tmQKV, stat_full, h * HD + p * 64, row_own);
          tma_load_2d(sStatB + p * 16384, &tmDO, stat_full, h * HD + p * 64, row_own);
        }
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % STAGES;
        const uint32_t use = it / STAGES;
        const int tile = MODE == 0 ? own + it : it;
        const int row = b * a.T + tile * 128;
        if (!mbar_wait(&empty[st], (use & 1) ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_EMPTY; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break;
        }
        mbar_expect_tx(&full[st], 2 * TILE_BYTES);
#pragma unroll
        for (int p = 0; p < PANELS; ++p) {
          if (MODE == 0) {
            tma_load_2d(sStrX + st * TILE_BYTES + p * 16384, &tmQKV, &full[st], h * HD + p * 64, row);
            tma_load_2d(sStrY + st * TILE_BYTES + p * 16384, &tmDO, &full[st], h * HD + p * 64, row);
          } else {
            tma_load_2d(sStrX + st * TILE_BYTES + p * 16384, &tmQKV, &full[st],
                        d_model + h * HD + p * 64, row);
            tma_load_2d(sStrY + st * TILE_BYTES + p * 16384, &tmQKV, &full[st],
                        2 * d_model + h * HD + p * 64, row);
          }
        }
      }
    }
  } else if (warp == BWD_MMA_WARP) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(stat_full, 0, abort_flag);
      // group 1: S = Q K^T, dP = dO V^T
      auto issue_sdp = [&](int it) {
        const int st = it % STAGES;
        if (!mbar_wait(&full[st], (it / STAGES) & 1, abort_flag)) return false;
        if (it > 0 && !mbar_wait(sdp_empty, (it - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t x = smem_u32(sStrX + st * TILE_BYTES), y = smem_u32(sStrY + st * TILE_BYTES);
        const uint32_t sa = smem_u32(sStatA), sb = smem_u32(sStatB);
        const uint32_t q = MODE == 0 ? x : sa, kk = MODE == 0 ? sa : x;
        const uint32_t dO = MODE == 0 ? y : sb, vv = MODE == 0 ? sb : y;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16(tS, make_sdesc_sw128(q + off, 16, 1024), make_sdesc_sw128(kk + off, 16, 1024),
                    IDESC_S, k > 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_bf16(tDP, make_sdesc_sw128(dO + off, 16, 1024), make_sdesc_sw128(vv + off, 16, 1024),
                    IDESC_S, k > 0);
        }
        umma_commit(sdp_full);
        return true;
      };
      // group 2: the accumulating products
      auto issue_acc = [&](int it) {
        const int st = it % STAGES;
        if (!mbar_wait(pds_full, it & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t x = smem_u32(sStrX + st * TILE_BYTES), y = smem_u32(sStrY + st * TILE_BYTES);
        const uint32_t p0 = smem_u32(sP), ds0 = smem_u32(sDS);
        if (MODE == 0) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {   // contraction over 128 query rows
            umma_bf16(tAcc0, make_sdesc_sw128(p0 + k * 2048, 16384, 1024),
                      make_sdesc_sw128(y + k * 2048, 16384, 1024), IDESC_T, (it > 0 || k > 0));
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            umma_bf16(tAcc1, make_sdesc_sw128(ds0 + k * 2048, 16384, 1024),
                      make_sdesc_sw128(x + k * 2048, 16384, 1024), IDESC_T, (it > 0 || k > 0));
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {   // contraction over 128 keys
            umma_bf16(tAcc0, make_sdesc_sw128(ds0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                      make_sdesc_sw128(x + k * 2048, 16384, 1024), IDESC_DQ, (it > 0 || k > 0));
          }
        }
        umma_commit(&empty[st]);
        umma_commit(pds_empty);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (STAGES > 1 && it + 1 < n_iter) { ok = issue_sdp(it + 1); if (!ok) break; }
        ok = issue_acc(it);
        if (!ok) break;
        if (STAGES == 1 && it + 1 < n_iter) ok = issue_sdp(it + 1);
      }
      if (ok) umma_commit(acc_full);
      else { *abort_flag = ST_TIMEOUT_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else {
    // ------------------------------------------------------------ math warps
    // warp w: TMEM lane quarter w & 3 (query rows 32*(w&3)..), key columns 32*(w>>2)..+31
    const int r = (warp & 3) * 32 + lane;
    const int cb = warp >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    const float dscale = dropout_scale(a.thr16);
    const long long bh = static_cast<long long>(b) * a.H + h;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int qi = MODE == 0 ? own + it : own;     // query tile
      const int kj = MODE == 0 ? own : it;           // key tile
      const int q_idx = qi * 128 + r;
      const bool q_ok = q_idx < a.T;
      const float lse_l2 = q_ok ? a.lse[bh * a.T + q_idx] * LOG2E : 0.f;
      const float dlt = q_ok ? a.delta[bh * a.T + q_idx] : 0.f;
      const bool diag = (qi == kj);
      const uint64_t row_elem0 = (static_cast<uint64_t>(bh) * a.T + q_idx) * a.T + kj * 128 + cb * 32;
      if (!mbar_wait(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      if (it > 0 && !mbar_wait(pds_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {      // two 16-column pieces keep the register count low
        const int col0 = cb * 32 + hf * 16;
        uint32_t sv[16], dv[16];
        tmem_ld16(tS + lane_addr + col0, sv);
        tmem_ld16(tDP + lane_addr + col0, dv);
        tmem_ld_wait();
        float p[16], ds[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool live = q_ok && (!diag || (col0 + i) <= r);
          p[i] = live ? ex2_fast(__uint_as_float(sv[i]) * sl2 - lse_l2) : 0.f;
          ds[i] = __uint_as_float(dv[i]);
        }
        if (a.thr16) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint64_t e0 = row_elem0 + hf * 16 + g * 8;
            const uint32_t keep = a.drop_mask
                ? (q_ok ? (a.drop_mask[e0 >> 5] >> (e0 & 31)) & 0xffu : 0u)
                : dropout_keep8(salted(a.seed, a.salt), a.stream_id, e0 >> 3, a.thr16);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const bool kp = (keep >> i) & 1u;
              const float pd = kp ? p[g * 8 + i] * dscale : 0.f;          // dropped P (for dV)
              const float dpe = kp ? ds[g * 8 + i] * dscale : 0.f;        // grad wrt softmax prob
              ds[g * 8 + i] = p[g * 8 + i] * (dpe - dlt) * a.scale;
              p[g * 8 + i] = pd;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) ds[i] = p[i] * (ds[i] - dlt) * a.scale;
        }
        const uint32_t poff = (col0 >> 6) * 16384;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t off = poff + sw128_chunk(r, ((col0 & 63) >> 3) + g);
          uint4 w;
          if (MODE == 0) {
            w.x = pack_bf16x2(p[g * 8 + 0], p[g * 8 + 1]); w.y = pack_bf16x2(p[g * 8 + 2], p[g * 8 + 3]);
            w.z = pack_bf16x2(p[g * 8 + 4], p[g * 8 + 5]); w.w = pack_bf16x2(p[g * 8 + 6], p[g * 8 + 7]);
            *reinterpret_cast<uint4*>(sP + off) = w;
          }
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
    }
    if (ok && !mbar_wait(acc_full, 0, abort_flag)) ok = false;
    if (!ok) { *abort_flag = ST_TIMEOUT_TMEM_FULL; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
    if (ok) {
      tc_fence_after();
      const int t_idx = own * 128 + r;   // row of the owned tile (key row in MODE 0, query row in MODE 1)
      __nv_bfloat16* base = a.dqkv + (static_cast<long long>(b) * a.T + t_idx) * (3 * d_model) + h * HD;
      constexpr int NACC = MODE == 0 ? 2 : 1;
      constexpr int CH = HD / 32;        // 32-column chunks per accumulator
      // MODE 0: acc0 = dV -> third block, acc1 = dK -> second block.  MODE 1: acc0 = dQ -> first.
      for (int g = cb; g < NACC * CH; g += 4) {
        const int which = g / CH, c = g % CH;
        const uint32_t tacc = which == 0 ? tAcc0 : tAcc1;
        __nv_bfloat16* dst = base + (MODE == 0 ? (which == 0 ? 2 * d_model : d_model) : 0);
        uint32_t v[32];
        tmem_ld32(tacc + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (t_idx < a.T) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BWD_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace ab

// ------------------------------------------------------------------------------------ host side
namespace ab {
int launch_attn_bwd_fused64(const CUtensorMap& tq, const CUtensorMap& td, const AttnBwdArgs& a,
                            cudaStream_t stream);   // attn_bwd_fused.cu

template <int HD>
static int launch_attn_fwd(const CUtensorMap& tm, const AttnArgs& a, cudaStream_t stream) {
  // output map: boxes of 32 rows x HD/2 columns (one math warp's share of a query tile)
  CUtensorMap tmo;
  const int rc_o = make_tmap_2d_sw(&tmo, a.out, (uint64_t)a.B * a.T, (uint64_t)a.H * HD, (uint64_t)a.H * HD,
                                   32, HD / 2, 2, HD);   // HD/2 bf16 columns = HD bytes per row
  if (rc_o) return rc_o;
  constexpr int SMEM = 5 * 128 * HD * 2 + 128 * 128 * 2 + 1024;
  auto kern = attn_fwd_kernel<HD>;
  static PerDeviceOnce attr;
  if (attr.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    // two CTAs per SM only fit when the SM is configured for its largest shared-memory carve-out
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    attr.mark_device();
  }
  dim3 grid((a.T + 127) / 128, a.H, a.B);
  launch_chained(kern, grid, dim3(FWD_THREADS), SMEM, stream, tm, tmo, a);
  return (int)cudaGetLastError();
}

template <int HD, int MODE>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& td, const AttnBwdArgs& a,
                           cudaStream_t stream) {
  constexpr int STAGES = HD <= 64 ? 2 : 1;
  constexpr int SMEM = (2 + 2 * STAGES) * 128 * HD * 2 + 2 * 128 * 128 * 2 + 256;
  auto kern = attn_bwd_kernel<HD, MODE>;
  static PerDeviceOnce attr;
  if (attr.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr.mark_device();
  }
  dim3 grid((a.T + 127) / 128, a.H, a.B);
  launch_chained(kern, grid, dim3(BWD_THREADS), SMEM, stream, tq, td, a);
  return (int)cudaGetLastError();
}
}  // namespace ab

extern "C" {

// qkv: bf16 [B*T, 3*H*hd]; out: bf16 [B*T, H*hd]; lse: fp32 [B,H,T] (may be null).
// hd must be 64 or 128.  With dropout (thr16 > 0) T must be a multiple of 8.
// drop_mask (optional): uint32 [B,H,T,T/32], receives the dropout keep bits (needs T % 32 == 0).
int ab_attn_fwd(const void* qkv, void* out, float* lse, unsigned int* drop_mask, int B, int T, int H,
                int hd, float scale, unsigned long long seed, unsigned int stream_id,
                unsigned int thr16, int* status, cudaStream_t stream) {
  using namespace ab;
  if ((hd != 64 && hd != 128) || B <= 0 || T <= 0 || (thr16 && (T & 7))) return -1;
  if (drop_mask && (T & 31)) return -1;
  CUtensorMap tm;
  int rc = make_tmap_2d(&tm, qkv, (uint64_t)B * T, 3ull * H * hd, 3ull * H * hd, 128, 64, 2, true);
  if (rc) return rc;
  AttnArgs a;
  a.B = B; a.T = T; a.H = H; a.hd = hd; a.scale = scale; a.seed = seed; a.stream_id = stream_id;
  a.thr16 = thr16; a.out = (__nv_bfloat16*)out; a.lse = lse; a.status = status; a.salt = seed_salt_ptr();
  a.drop_mask = drop_mask;
  return hd == 64 ? launch_attn_fwd<64>(tm, a, stream) : launch_attn_fwd<128>(tm, a, stream);
}

// delta: fp32 scratch [B,H,T] owned by the caller.  drop_mask (optional): the keep bits the forward
// pass wrote.  dq_acc (optional, hd == 64): fp32 [B*T, H*hd] accumulator that must be all zero on
// entry and is all zero again on return; when given, the single-kernel backward runs.
int ab_attn_bwd(const void* qkv, const void* out, const float* lse, const void* dout, void* dqkv,
                float* delta, const unsigned int* drop_mask, float* dq_acc, int B, int T, int H, int hd,
                float scale, unsigned long long seed, unsigned int stream_id, unsigned int thr16,
                int* status, cudaStream_t stream) {
  using namespace ab;
  if ((hd != 64 && hd != 128) || B <= 0 || T <= 0 || (thr16 && (T & 7))) return -1;
  if (drop_mask && (T & 31)) return -1;
  CUtensorMap tq, td;
  int rc = make_tmap_2d(&tq, qkv, (uint64_t)B * T, 3ull * H * hd, 3ull * H * hd, 128, 64, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&td, dout, (uint64_t)B * T, (uint64_t)H * hd, (uint64_t)H * hd, 128, 64, 2, true);
  if (rc) return rc;
  const long long n = (long long)B * T * H * (hd / 8);
  launch_chained(attn_delta_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                 (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, B, T, H, hd);
  AttnBwdArgs a;
  a.B = B; a.T = T; a.H = H; a.hd = hd; a.scale = scale; a.seed = seed; a.stream_id = stream_id;
  a.thr16 = thr16; a.lse = lse; a.delta = delta; a.dqkv = (__nv_bfloat16*)dqkv; a.status = status;
  a.salt = seed_salt_ptr();
  a.drop_mask = drop_mask; a.dq_acc = dq_acc;
  if (hd == 64 && dq_acc) return launch_attn_bwd_fused64(tq, td, a, stream);
  if (hd == 64) {
    rc = launch_attn_bwd<64, 0>(tq, td, a, stream);
    if (rc) return rc;
    return launch_attn_bwd<64, 1>(tq, td, a, stream);
  }
  rc = launch_attn_bwd<128, 0>(tq, td, a, stream);
  if (rc) return rc;
  return launch_attn_bwd<128, 1>(tq, td, a, stream);
}
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (see attn_static.cuh for who needs it and why).
#include <atomic>

#include "attn_static.cuh"

namespace ab {
// Scratch for `delta`.  In host code this name is only a handle; the device address is looked up
// per device below.
static __device__ __align__(256) float g_attn_static_delta[AB_ATTN_STATIC_MAX_ROWS];
// Per-device cache of the array's device address.  Host threads may fill an entry concurrently;
// they all store the same value, and the atomic keeps the store and the loads untorn.
static std::atomic<float*> g_attn_static_ptr[64];
}  // namespace ab

extern "C" int ab_attn_bwd_static(const void* qkv, const void* out, const float* lse,
                                  const void* dout, void* dqkv, const unsigned int* drop_mask, int B,
                                  int T, int H, int hd, float scale, unsigned long long seed,
                                  unsigned int stream_id, unsigned int thr16, int* status,
                                  cudaStream_t stream) {
  using namespace ab;
  if (B <= 0 || T <= 0 || H <= 0) return -1;
  if (static_cast<long long>(B) * H * T > AB_ATTN_STATIC_MAX_ROWS) return -10;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -11;
  float* scratch = g_attn_static_ptr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // once per device, with that device current: turn the symbol into a device pointer
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_static_delta);
    if (e != cudaSuccess) return (int)e;
    scratch = static_cast<float*>(p);
    g_attn_static_ptr[dev].store(scratch, std::memory_order_release);
  }
  return ab_attn_bwd(qkv, out, lse, dout, dqkv, scratch, drop_mask, nullptr, B, T, H, hd,
                     scale, seed, stream_id, thr16, status, stream);
}
