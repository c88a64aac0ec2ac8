// Fused output-embedding GEMM + cross entropy for training (forward and the gradient of the
// logits in one launch; the logits themselves never reach memory).
//
//   logits[m, :] = h[m, :] . wte^T        (bf16 operands, fp32 accumulation in TMEM)
//   loss        += sum over rows with label >= 0 of  logsumexp(logits[m, :]) - logits[m, label[m]]
//   dlogits[m, n] = (softmax(logits[m, :])[n] - [n == label[m]]) * coef / n_valid   (0 for ignored rows)
//
// A CTA owns 128 rows at a time and walks the vocabulary in tiles of 256 columns, TWICE: the first
// sweep keeps a running maximum and sum of exponentials per row (online softmax across the N
// tiles) and picks up the label's logit; the second sweep recomputes every tile on the tensor
// cores and turns it straight into the bf16 gradient tile, which leaves through TMA stores and is
// the operand of the two GEMMs that follow (d h = dlogits . wte, d wte += dlogits^T . h).  The
// second sweep costs one more pass of a GEMM that is under 1 % of the step; in exchange the
// [M, V] logits are neither written, re-read nor rounded to bf16 before the softmax.
//
// Same pipeline as the plain GEMM (gemm_tc.cu): warp 0 TMA producer, warp 1 MMA issuer, 16 epilogue
// warps (four per TMEM lane quarter, 64 columns each), two accumulators in TMEM so the epilogue of
// tile i overlaps the MMAs of tile i + 1.  Every wait is bounded and reports through `status`.
#include "gemm_core.cuh"

namespace ab {

constexpr int LC_BN = 256;
constexpr int LC_STAGES = 3;      // 3 x 48 KB operand stages leave room for the row statistics

struct LmCeArgs {
  int M, V, K;
  const int* labels;      // [M], < 0 = ignored
  const int* n_valid;     // device scalar: rows with a label
  float coef;
  float* loss_acc;        // += sum of the rows' negative log likelihoods
  int* status;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
lmhead_ce_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmOut, const LmCeArgs g) {
  griddep_enter();
  constexpr int BN = LC_BN, STAGES = LC_STAGES;
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  constexpr float L2E = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_out = smem + STAGES * STAGE_BYTES;                 // 2 KB per epilogue warp
  // row statistics shared between the sweeps: [2 unit parities][3: max, sum, label logit][4 parts][128 rows]
  float* s_stat = reinterpret_cast<float*>(stage_out + NUM_EPI_WARPS * 2048);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_stat + 2 * 3 * 4 * BM);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* stat_bar = bars + 2 * STAGES + 4;       // the 16 epilogue warps meet here once per unit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], NUM_EPI_WARPS); }
    mbar_init(stat_bar, NUM_EPI_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmOut);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (g.M + BM - 1) / BM;
  const int n_tiles = (g.V + BN - 1) / BN;
  const int kb_total = (g.K + BK - 1) / BK;
  const int tiles_per_unit = 2 * n_tiles;                  // two sweeps over the vocabulary

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < m_tiles && ok; u += gridDim.x) {
        const int m0 = u * BM;
        for (int t = 0; t < tiles_per_unit && ok; ++t) {
          const int n0 = (t % n_tiles) * BN;
          for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
              *abort_flag = ST_TIMEOUT_EMPTY;
              atomicCAS(g.status, 0, ST_TIMEOUT_EMPTY);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
            tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m0);
            tma_load_2d(sa + A_BYTES, &tmB, &full_bar[stage], kb * BK, n0);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < m_tiles && ok; u += gridDim.x) {
        for (int t = 0; t < tiles_per_unit && ok; ++t, ++it) {
          const int ab = it & 1;
          if (!mbar_wait(&tempty_bar[ab], acc_phase[ab] ^ 1, abort_flag)) {
            *abort_flag = ST_TIMEOUT_TMEM_EMPTY;
            atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_EMPTY);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + ab * BN;
          for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
              *abort_flag = ST_TIMEOUT_FULL;
              atomicCAS(g.status, 0, ST_TIMEOUT_FULL);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint32_t sb = sa + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = make_sdesc_sw128(sa + k * UMMA_K * 2, 16, 1024);
              const uint64_t bdesc = make_sdesc_sw128(sb + k * UMMA_K * 2, 16, 1024);
              umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&tfull_bar[ab]);
          acc_phase[ab] ^= 1;
        }
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue
    const int e = warp - 2;
    const int quad = warp & 3;           // TMEM lane quarter this warp may read
    const int part = e >> 2;             // which 64 of the tile's 256 columns
    constexpr int COLS_PER_WARP = BN / 4;
    uint8_t* my_stage = stage_out + e * 2048;
    const int rloc = quad * 32 + lane;   // row inside the 128-row tile
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    const int nval = __ldg(g.n_valid);
    const float gscale = nval > 0 ? g.coef / static_cast<float>(nval) : 0.f;
    float loss_local = 0.f;
    bool ok = true;
    uint32_t unit_it = 0;
    for (int u = blockIdx.x; u < m_tiles && ok; u += gridDim.x, ++unit_it) {
      float* s_m = s_stat + (unit_it & 1) * (3 * 4 * BM);     // double-buffered by unit parity: a warp can
      float* s_l = s_m + 4 * BM;                              // only overwrite a buffer after every warp
      float* s_lab = s_l + 4 * BM;                            // has passed the meeting that follows its use
      const int m = u * BM + rloc;
      const int m0w = u * BM + quad * 32;
      const bool row_in = m < g.M;
      const int label = row_in ? __ldg(g.labels + m) : -1;
      float rm = -INFINITY, rl = 0.f, rlab = -INFINITY, lse = 0.f;
      for (int t = 0; t < tiles_per_unit; ++t, ++it) {
        const int ab = it & 1;
        const int sweep = t / n_tiles;
        const int nbase = (t % n_tiles) * BN + part * COLS_PER_WARP;
        if (sweep == 1 && t == n_tiles) {
          // between the sweeps: the four column parts of a row share their statistics
          s_m[part * BM + rloc] = rm;
          s_l[part * BM + rloc] = rl;
          s_lab[part * BM + rloc] = rlab;
          __syncwarp();
          if (lane == 0) mbar_arrive(stat_bar);
          if (!mbar_wait(stat_bar, unit_it & 1, abort_flag)) {     // bounded, and it sees another warp's abort
            *abort_flag = ST_TIMEOUT_MISC;
            atomicCAS(g.status, 0, ST_TIMEOUT_MISC);
            ok = false;
            break;
          }
          float M4 = -INFINITY;
#pragma unroll
          for (int p = 0; p < 4; ++p) M4 = fmaxf(M4, s_m[p * BM + rloc]);
          float L4 = 0.f, lab = -INFINITY;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float mp = s_m[p * BM + rloc];
            if (mp != -INFINITY) L4 += s_l[p * BM + rloc] * ex2_fast((mp - M4) * L2E);
            lab = fmaxf(lab, s_lab[p * BM + rloc]);
          }
          lse = M4 + logf(L4);
          if (part == 0 && label >= 0) loss_local += lse - lab;
        }
        if (!mbar_wait(&tfull_bar[ab], acc_phase[ab], abort_flag)) {
          *abort_flag = ST_TIMEOUT_TMEM_FULL;
          atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_FULL);
          ok = false;
          break;
        }
        acc_phase[ab] ^= 1;
        tc_fence_after();
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ab * BN + part * COLS_PER_WARP;
#pragma unroll 1
        for (int rd = 0; rd < COLS_PER_WARP / 16; ++rd) {
          const int n0 = nbase + rd * 16;
          if (n0 >= g.V) break;                             // warp-uniform
          uint32_t r[16];
          tmem_ld16(taddr + rd * 16, r);
          if (sweep == 1 && lane == 0) tma_store_wait_read<0>();   // staging tile free again
          __syncwarp();
          tmem_ld_wait();
          if (sweep == 0) {
            float tm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float v = (n0 + j < g.V) ? __uint_as_float(r[j]) : -INFINITY;
              tm = fmaxf(tm, v);
              if (n0 + j == label) rlab = v;
            }
            const float m_new = fmaxf(rm, tm);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (n0 + j < g.V) s += ex2_fast((__uint_as_float(r[j]) - m_new) * L2E);
            rl = rl * ex2_fast((rm - m_new) * L2E) + s;
            rm = m_new;
          } else {
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
              float p[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int n = n0 + grp * 8 + j;
                float v = 0.f;
                if (label >= 0 && n < g.V) {
                  v = ex2_fast((__uint_as_float(r[grp * 8 + j]) - lse) * L2E) * gscale;
                  if (n == label) v -= gscale;
                }
                p[j] = v;
              }
              // 16 bf16 columns = 32-byte rows, 32B swizzle: chunk index ^= (row >> 2) & 1
              const uint32_t off = lane * 32 + ((grp ^ ((lane >> 2) & 1)) << 4);
              uint4 o;
              o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
              o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
              *reinterpret_cast<uint4*>(my_stage + off) = o;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmOut, my_stage, n0, m0w);
              tma_store_commit();
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[ab]);
      }
    }
    if (lane == 0) tma_store_wait<0>();
    // loss: only the part-0 warps hold row losses
#pragma unroll
    for (int o = 16; o; o >>= 1) loss_local += __shfl_xor_sync(0xffffffffu, loss_local, o);
    if (lane == 0 && part == 0 && loss_local != 0.f) atomicAdd(g.loss_acc, loss_local);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace ab

// h: [M, K] bf16 (final hidden states), wte: [V, K] bf16, labels: [M] int (already shifted, < 0 =
// ignored), dlogits: [M, V] bf16 out.  K, V multiples of 8.
extern "C" int ab_lmhead_ce(const void* h, long long ldh, const void* wte, long long ldw, const int* labels,
                            const int* n_valid, float coef, void* dlogits, long long ldo, float* loss_acc,
                            int M, int V, int K, int max_ctas, int* status, cudaStream_t stream) {
  using namespace ab;
  if (M <= 0 || V <= 0 || K <= 0 || (V & 7) || (K & 7) || (ldh & 7) || (ldw & 7) || (ldo & 7) || !status) return -1;
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(wte) | reinterpret_cast<uintptr_t>(dlogits)) & 15)
    return -3;
  CUtensorMap tmA, tmB, tmOut;
  int rc = make_tmap_2d(&tmA, h, M, K, ldh, BM, BK, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, wte, V, K, ldw, LC_BN, BK, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d_sw(&tmOut, dlogits, M, V, ldo, 32, 16, 2, 32);
  if (rc) return rc;
  LmCeArgs g;
  g.M = M; g.V = V; g.K = K; g.labels = labels; g.n_valid = n_valid; g.coef = coef; g.loss_acc = loss_acc;
  g.status = status;
  constexpr int SMEM = 1024 + LC_STAGES * (BM * BK * 2 + LC_BN * BK * 2) + NUM_EPI_WARPS * 2048 + 2 * 3 * 4 * BM * 4 + 256;
  static PerDeviceOnce attr_set;
  if (attr_set.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(lmhead_ce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set.mark_device();
  }
  if (max_ctas <= 0) max_ctas = 148;
  const int m_tiles = (M + BM - 1) / BM;
  const int grid = m_tiles < max_ctas ? m_tiles : max_ctas;
  launch_chained(lmhead_ce_kernel, dim3(grid), dim3(NUM_THREADS), SMEM, stream, tmA, tmB, tmOut, g);
  return static_cast<int>(cudaGetLastError());
}
