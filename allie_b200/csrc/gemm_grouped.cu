// Grouped bf16 GEMM for the expert layers of a mixture-of-experts model: ONE persistent CTA-pair
// launch (tcgen05.mma.cta_group::2, 256 x 256 tiles, TMA-fed, TMEM double-buffered; the same
// pipeline as gemm_bf16_tcgen05_pair_kernel in gemm_tc.cu) runs a projection for all local experts.
//
//   mode 1  C[g] = A[g] * B[g] (+ bias[g], GELU ...) over the live rows of every group.  The work
//           list is built on the device from the per-group row counts, so tiles past a group's
//           live rows are never scheduled, and a launch sized for the capacity costs what the
//           routed tokens cost.
//   mode 2  C[g] += A[g]^T * B[g], contraction over the group's live rows (weight gradients).
//
// Two things make it a fused compute + collective kernel in the expert-parallel forward / backward:
//   * Arrival counters.  Rows of A are written by other GPUs (the dispatch kernels store token
//     rows straight into this rank's receive buffer and then increment the counter of the 128-row
//     block with release semantics).  The TMA producer of a tile waits, bounded, until the blocks
//     it is about to read are complete, so the GEMM starts on the tiles that have arrived while
//     later ones are still in flight.
//   * Scattering epilogue.  The down projection does not write its result locally: every epilogue
//     warp stages its 32 x 64 bf16 block in shared memory and then stores each row into the combine
//     buffer of the rank the token came from, at its return address (128 contiguous bytes per row
//     and warp, plain peer stores).  The last CTA to finish releases a phase flag to every rank;
//     the consumer kernel on the source rank waits for all of them.
#include "gemm_core.cuh"
#include "gemm_grouped.cuh"
#include "nvl_sync.cuh"

namespace ab {

constexpr int MAX_GROUPS = 64;

struct GroupedArgs {
  int groups, cap, mode;
  const int* rows;
  const unsigned int* tile_ready;
  const int* ret;
  NvlPeers dst, flags;
  int phase;
  uint32_t epoch;
  int rank, world;
  unsigned int* ticket;
};

__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Bounded wait until an arrival counter reaches `need`.  One thread.
__device__ __forceinline__ bool wait_rows(const unsigned int* ctr, unsigned int need,
                                          volatile int* abort_flag) {
  if (need == 0) return true;
  if (ld_acquire_sys(ctr) >= need) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (ld_acquire_sys(ctr) < need) {
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > AB_SPIN_CYCLES) return false;
    }
  }
  return true;
}

// Epilogue of the scattering down projection: 64 bf16 columns of 32 rows go through the warp's
// staging tile (128-byte rows, 128B-swizzle pattern so the row-wise writes and the chunk-wise
// reads are both conflict-free) and leave as one 128-byte segment per row to `dst_row` (null:
// the row is not live).
__device__ __forceinline__ void epilogue_drain_scatter64(const GemmArgs& g, uint32_t taddr, int m,
                                                         int nbase, bool row_ok, uint8_t* stg, int lane,
                                                         int bias_off, __nv_bfloat16* dst_row) {
  __syncwarp();
#pragma unroll 1
  for (int rd = 0; rd < 4; ++rd) {
    const int n0 = nbase + rd * 16;
    if (n0 >= g.N) break;
    uint32_t r[16];
    tmem_ld16(taddr + rd * 16, r);
    tmem_ld_wait();
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      const int n = n0 + grp * 8;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[grp * 8 + j]);
      uint4 pre = make_uint4(0, 0, 0, 0);
      epilogue_math8(g, v, pre, m, n, row_ok && n < g.N, true, bias_off);
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
      const int c = rd * 2 + grp;
      *reinterpret_cast<uint4*>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) = o;
    }
  }
  __syncwarp();
  // four rows per pass: lane -> (row = 4 * it + lane / 8, 16-byte chunk = lane % 8)
  const unsigned long long mine = reinterpret_cast<unsigned long long>(dst_row);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3), c = lane & 7;
    const unsigned long long p = __shfl_sync(0xffffffffu, mine, row);
    const int n = nbase + c * 8;
    if (p && n < g.N) {
      const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 128 + ((c ^ (row & 7)) << 4));
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + n) = val;
    }
  }
}

template <bool A_MN, bool B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmOut,
                         const __grid_constant__ CUtensorMap tmAux, const GemmArgs g,
                         const GroupedArgs ga) {
  static_assert(MODE == 1 ? !A_MN : (A_MN && B_MN), "mode 1: K-major A; mode 2: both MN-major");
  constexpr int STAGES = PAIR_STAGES;
  constexpr int BN = PAIR_BN;
  constexpr int HALF_N = BN / 2;
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = HALF_N * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_out = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + NUM_EPI_WARPS * PAIR_WARP_STAGING);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_rows = reinterpret_cast<int*>(tmem_slot + 2);        // [MAX_GROUPS] live rows, clipped to cap
  int* s_tile0 = s_rows + MAX_GROUPS;                         // [MAX_GROUPS + 1] first 256-row tile of a group

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 2 * NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmOut);
    if (g.ep.act == 1) tma_prefetch_desc(&tmAux);
    int acc = 0;
    for (int i = 0; i < ga.groups; ++i) {
      const int r = max(0, min(ga.cap, __ldg(ga.rows + i)));
      s_rows[i] = r;
      s_tile0[i] = acc;
      acc += (r + 2 * BM - 1) / (2 * BM);
    }
    s_tile0[ga.groups] = acc;
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_tiles = (g.N + BN - 1) / BN;
  const int m_tiles2 = (g.M + 2 * BM - 1) / (2 * BM);          // mode 2: tiles of the per-group output
  const int per_group2 = m_tiles2 * n_tiles;
  const int num_units = MODE == 1 ? s_tile0[ga.groups] * n_tiles : ga.groups * per_group2;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // unit -> (group, first row of the pair's tile inside the group, first column, K blocks)
  auto decode = [&](int u, int& grp, int& mrow0, int& ncol0, int& kb_total) {
    if constexpr (MODE == 1) {
      const int mtg = u / n_tiles;
      ncol0 = (u % n_tiles) * BN;
      int gi = 0;
      while (gi + 1 < ga.groups && s_tile0[gi + 1] <= mtg) ++gi;
      grp = gi;
      mrow0 = (mtg - s_tile0[gi]) * (2 * BM);
      kb_total = (g.K + BK - 1) / BK;
    } else {
      grp = u / per_group2;
      const int t = u % per_group2;
      mrow0 = (t / n_tiles) * (2 * BM);
      ncol0 = (t % n_tiles) * BN;
      kb_total = ((s_rows[grp] + 127) & ~127) / BK;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        int grp, mrow0, ncol0, kb_total;
        decode(u, grp, mrow0, ncol0, kb_total);
        const int n0 = ncol0 + rank * HALF_N;
        if constexpr (MODE == 1) {
          if (ga.tile_ready) {
            // my 128 rows of A: complete once every live row in them has arrived
            const int first = mrow0 + rank * BM;
            const int need = max(0, min(BM, s_rows[grp] - first));
            if (!wait_rows(ga.tile_ready + (grp * ga.cap + first) / BM, need, abort_flag)) {
              *abort_flag = ST_TIMEOUT_PEER;
              atomicCAS(g.status, 0, ST_TIMEOUT_PEER);
              ok = false;
              break;
            }
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < kb_total; ++kb) {
          const int k0 = kb * BK;
          if constexpr (MODE == 2) {
            if (ga.tile_ready && (k0 % BM) == 0) {
              const int need = max(0, min(BM, s_rows[grp] - k0));
              if (!wait_rows(ga.tile_ready + (grp * ga.cap + k0) / BM, need, abort_flag)) {
                *abort_flag = ST_TIMEOUT_PEER;
                atomicCAS(g.status, 0, ST_TIMEOUT_PEER);
                ok = false;
                break;
              }
              fence_proxy_async_all();
            }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            *abort_flag = ST_TIMEOUT_EMPTY;
            atomicCAS(g.status, 0, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          if constexpr (MODE == 1) {
            tma_load_2d_pair(sa, &tmA, fb, k0, grp * ga.cap + mrow0 + rank * BM);
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tmB, fb, k0, grp * g.N + n0);
            } else {
#pragma unroll
              for (int i = 0; i < HALF_N / 64; ++i)
                tma_load_2d_pair(sb + i * (BK * 128), &tmB, fb, n0 + i * 64, grp * g.K + k0);
            }
          } else {
            const int y = grp * ga.cap + k0;
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d_pair(sa + i * (BK * 128), &tmA, fb, mrow0 + rank * BM + i * 64, y);
#pragma unroll
            for (int i = 0; i < HALF_N / 64; ++i)
              tma_load_2d_pair(sb + i * (BK * 128), &tmB, fb, n0 + i * 64, y);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16;
      constexpr uint32_t B_LBO = B_MN ? BK * 128 : 16;
      constexpr uint32_t A_KADV = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t B_KADV = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        int grp, mrow0, ncol0, kb_total;
        decode(u, grp, mrow0, ncol0, kb_total);
        if (kb_total == 0) continue;
        const int ab = it & 1;
        ++it;
        if (!mbar_wait(&tempty_bar[ab], acc_phase[ab] ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_TMEM_EMPTY;
          atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_EMPTY);
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
            const uint64_t adesc = make_sdesc_sw128(sa + k * A_KADV, A_LBO, 1024);
            const uint64_t bdesc = make_sdesc_sw128(sb + k * B_KADV, B_LBO, 1024);
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(mapa_shared(eb, 0));
          umma_commit_pair(mapa_shared(eb, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t tb = smem_u32(&tfull_bar[ab]);
        umma_commit_pair(mapa_shared(tb, 0));
        umma_commit_pair(mapa_shared(tb, 1));
        acc_phase[ab] ^= 1;
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue (both CTAs)
    const int e = warp - 2;
    const int quad = warp & 3;
    const int part = e >> 2;
    constexpr int COLS_PER_WARP = BN / 4;
    uint8_t* my_stage = stage_out + e * PAIR_WARP_STAGING;
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    for (int u = pair_id; u < num_units; u += num_pairs) {
      int grp, mrow0, ncol0, kb_total;
      decode(u, grp, mrow0, ncol0, kb_total);
      if (kb_total == 0) continue;
      const int ab = it & 1;
      ++it;
      const int mrow_w = mrow0 + rank * BM + quad * 32;        // first row of this warp, inside the group
      const int mrow = mrow_w + lane;
      const int nbase = ncol0 + part * COLS_PER_WARP;
      if (!mbar_wait(&tfull_bar[ab], acc_phase[ab], abort_flag)) {
        *abort_flag = ST_TIMEOUT_TMEM_FULL;
        atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      acc_phase[ab] ^= 1;
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ab * BN + part * COLS_PER_WARP;
      if constexpr (MODE == 1) {
        const int live = s_rows[grp];
        // whole 128-row blocks are written: the rows between the live ones and the next multiple
        // of 128 take part in the weight-gradient contractions and must not keep stale values
        if (mrow_w < ((live + 127) & ~127)) {
          const int row_g = grp * ga.cap + mrow;               // row in A / out / aux / ret
          const bool row_ok = mrow < live;
          if (ga.ret) {
            __nv_bfloat16* dst_row = nullptr;
            if (row_ok) {
              const int ra = __ldg(ga.ret + row_g);
              dst_row = static_cast<__nv_bfloat16*>(ga.dst.ptr[ra >> 24]) +
                        static_cast<long long>(ra & 0xffffff) * g.N;
            }
            epilogue_drain_scatter64(g, taddr, row_g, nbase, row_ok, my_stage, lane, grp * g.N, dst_row);
          } else {
            epilogue_drain_wide<COLS_PER_WARP>(g, tmOut, tmAux, taddr, row_g, grp * ga.cap + mrow_w, nbase,
                                               row_ok, my_stage, lane, true, grp * g.N);
          }
        }
      } else {
        if (mrow_w < g.M)
          epilogue_drain_wide<COLS_PER_WARP>(g, tmOut, tmAux, taddr, grp * g.M + mrow, grp * g.M + mrow_w, nbase,
                                             mrow < g.M, my_stage, lane, true, grp * g.N);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[ab]), 0));
    }
    if (lane == 0) tma_store_wait<0>();
    if (ga.ret) __threadfence_system();        // this warp's peer stores are out before the CTA reports
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (ga.ret && warp == 2) {
    // the last CTA of the grid releases the phase to every rank
    int last = 0;
    if (lane == 0) {
      __threadfence_system();
      last = atomicAdd(ga.ticket, 1u) == gridDim.x - 1;
      if (last) *ga.ticket = 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last && lane < ga.world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(ga.flags.ptr[lane]) + ga.phase * FLAG_STRIDE + ga.rank, ga.epoch);
    }
  }
}

template <bool A_MN, bool B_MN, int MODE>
static int launch_grouped(const void* A, long long lda, const void* B, long long ldb, const GemmArgs& g,
                          const GroupedArgs& ga, int max_ctas, cudaStream_t stream) {
  constexpr int HALF_N = PAIR_BN / 2;
  CUtensorMap tmA, tmB, tmOut, tmAux;
  const AbGemmEpilogue& ep = g.ep;
  const uint64_t G = ga.groups, cap = ga.cap;
  const void* obase = ep.out ? ep.out : A;      // the scattering epilogue has no local output; the map is unused
  const long long oldo = ep.out ? ep.ldo : g.N;
  int rc;
  if (MODE == 1) {
    rc = make_tmap_2d(&tmA, A, G * cap, g.K, lda, BM, BK, 2, true);
    if (rc) return rc;
    if (!B_MN) rc = make_tmap_2d(&tmB, B, G * g.N, g.K, ldb, HALF_N, BK, 2, true);
    else       rc = make_tmap_2d(&tmB, B, G * g.K, g.N, ldb, BK, 64, 2, true);
    if (rc) return rc;
    if (ep.act == 1)  rc = make_tmap_2d_sw(&tmOut, obase, G * cap, g.N, oldo, 32, 32, 2, 64);
    else              rc = make_tmap_2d_sw(&tmOut, obase, G * cap, g.N, oldo, 32, 64, 2, 128);
    if (rc) return rc;
    if (ep.act == 1) {
      rc = make_tmap_2d_sw(&tmAux, ep.aux, G * cap, g.N, ep.ldaux, 32, 32, 2, 64);
      if (rc) return rc;
    } else {
      tmAux = tmOut;
    }
  } else {
    rc = make_tmap_2d(&tmA, A, G * cap, g.M, lda, BK, 64, 2, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, B, G * cap, g.N, ldb, BK, 64, 2, true);
    if (rc) return rc;
    rc = make_tmap_2d_sw(&tmOut, ep.out, G * g.M, g.N, ep.ldo, 32, 32, 4, 128);
    if (rc) return rc;
    tmAux = tmOut;
  }
  constexpr int SMEM = 1024 + PAIR_STAGES * (BM * BK * 2 + HALF_N * BK * 2) +
                       NUM_EPI_WARPS * PAIR_WARP_STAGING + 256 + (2 * MAX_GROUPS + 8) * 4;
  auto kern = gemm_grouped_pair_kernel<A_MN, B_MN, MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int n_tiles = (g.N + PAIR_BN - 1) / PAIR_BN;
  const long long units = MODE == 1 ? G * (cap / (2 * BM)) * n_tiles
                                    : G * ((g.M + 2 * BM - 1) / (2 * BM)) * n_tiles;
  int pairs = max_ctas / 2;
  if (pairs > units) pairs = static_cast<int>(units);
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, NUM_THREADS, SMEM, stream>>>(tmA, tmB, tmOut, tmAux, g, ga);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ab

extern "C" int ab_gemm_grouped_bf16(const void* A, long long lda, const void* B, int b_mn,
                                    long long ldb, int M, int N, int K, const AbGemmEpilogue* ep,
                                    const AbGroupedGemm* grp, int max_ctas, int* status,
                                    cudaStream_t stream) {
  using namespace ab;
  if (!ep || !grp || !status || !grp->rows) return -1;
  if (grp->groups < 1 || grp->groups > MAX_GROUPS || grp->cap < 2 * BM || (grp->cap % (2 * BM))) return -1;
  if (N <= 0 || (N & 7) || (lda & 7) || (ldb & 7)) return -1;
  if (ep->resid || ep->m_limit || ep->k_limit) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(ep->out) | reinterpret_cast<uintptr_t>(ep->aux)) & 15)
    return -3;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K; g.k_splits = 1; g.pdl = 0; g.ep = *ep; g.status = status; g.salt = seed_salt_ptr(); g.aux_tma = 0;
  GroupedArgs ga;
  ga.groups = grp->groups; ga.cap = grp->cap; ga.mode = grp->mode; ga.rows = grp->rows;
  ga.tile_ready = grp->tile_ready; ga.ret = grp->ret; ga.phase = grp->phase; ga.epoch = grp->epoch;
  ga.rank = grp->rank; ga.world = grp->world; ga.ticket = grp->ticket;
  for (int i = 0; i < MAX_RANKS; ++i) {
    ga.dst.ptr[i] = grp->peers[i];
    ga.flags.ptr[i] = grp->flags[i];
  }
  if (max_ctas <= 0) max_ctas = 148;
  if (max_ctas < 2) return -1;
  if (grp->mode == 1) {
    if (K <= 0 || (K % BK)) return -4;                  // a K block must not run into the next group's weights
    if (ep->out_fp32 || ep->accumulate) return -2;
    if (grp->ret) {
      if (ep->act || !grp->ticket || grp->world < 1 || grp->world > MAX_RANKS) return -2;
    } else {
      if (!ep->out || ((ep->ldo * 2) & 15)) return -4;
      if (ep->act == 1 && (!ep->aux || (ep->ldaux & 7))) return -4;
    }
    if (b_mn) return launch_grouped<false, true, 1>(A, lda, B, ldb, g, ga, max_ctas, stream);
    return launch_grouped<false, false, 1>(A, lda, B, ldb, g, ga, max_ctas, stream);
  }
  if (grp->mode == 2) {
    if (M <= 0 || (M % 32) || !ep->out_fp32 || !ep->accumulate || ep->act || ep->bias || grp->ret) return -2;
    if (!ep->out || ((ep->ldo * 4) & 15) || !b_mn) return -4;
    return launch_grouped<true, true, 2>(A, lda, B, ldb, g, ga, max_ctas, stream);
  }
  return -1;
}
