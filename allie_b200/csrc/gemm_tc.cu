// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   warp 0      : TMA producer   (cp.async.bulk.tensor into a STAGES-deep smem ring)
//   warp 1      : MMA issuer     (one thread issues tcgen05.mma; accumulators live in TMEM)
//   warps 2..17 : epilogue       (tcgen05.ld TMEM -> registers -> fused epilogue -> global);
//                 four warps per TMEM lane quarter, each owning a quarter of the tile's columns
//
// The 512 TMEM columns hold two 128 x BN fp32 accumulators, so the epilogue of
// work unit i overlaps the main loop of unit i+1.  Work units are
// (output tile, K split) pairs handed out round-robin to a grid of at most one
// CTA per SM.  Operands may be K-major or MN-major in memory (the UMMA
// descriptors express both), which covers forward (X*W), dgrad (dY*W^T) and
// wgrad (X^T*dY) of a layer whose weight is stored [in][out] without any
// transposed copies.  No TMA multicast is used anywhere.
#include "gemm_core.cuh"
#include <cstdlib>

namespace ab {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, int elem_bytes, bool swizzle128) {
  return make_tmap_2d_sw(out, base, rows, cols, ld, box_rows, box_cols, elem_bytes,
                         swizzle128 ? 128 : 0);
}

int make_tmap_2d_sw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows, uint32_t box_cols, int elem_bytes, int swizzle_bytes) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -100;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                   : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                   : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -200 - static_cast<int>(r);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmOut,
                         const __grid_constant__ CUtensorMap tmAux, const GemmArgs g) {
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;  // 256 or 512, power of two
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512 || TMEM_COLS == 128, "bad BN");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  // per-epilogue-warp staging tiles for the TMA stores: 2 KB each (32 rows x 16 columns of
  // fp32, or 32 x 16 bf16 output + 32 x 16 bf16 pre-activation)
  uint8_t* stage_out = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + NUM_EPI_WARPS * 2048);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmOut);
    if (g.ep.act == 1) tma_prefetch_desc(&tmAux);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  // the kernel behind this one in the stream may begin its own set-up now
  if (threadIdx.x == 0) griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // As a programmatic dependent this kernel may be running before its predecessor has finished:
  // only the weight operand B (and the set-up above) is touched before griddep_wait.  m_limit /
  // k_limit are device values of earlier kernels, so such launches are never made dependent.
  if (warp >= 2) griddep_wait();          // epilogue: residual / aux reads and every store come after

  const int Meff = g.ep.m_limit ? min(g.M, __ldg(g.ep.m_limit)) : g.M;
  const int Keff = g.ep.k_limit ? min(g.K, __ldg(g.ep.k_limit)) : g.K;
  const int m_tiles = (Meff + BM - 1) / BM;
  const int n_tiles = (g.N + BN - 1) / BN;
  const int kb_total = (Keff + BK - 1) / BK;
  const int kb_per = (kb_total + g.k_splits - 1) / g.k_splits;
  const int num_tiles = m_tiles * n_tiles;
  // units are ordered K-split-major: CTAs running at the same time work on the same K range of
  // different output tiles, so each operand slab is fetched from HBM once and shared through L2
  const int num_units = num_tiles * g.k_splits;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto load_b = [&](uint8_t* sb, uint64_t* bar, int k0, int n0) {
        if constexpr (!B_MN) {
          tma_load_2d(sb, &tmB, bar, k0, n0);
        } else {
#pragma unroll
          for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * (BK * 128), &tmB, bar, n0 + i * 64, k0);
        }
      };
      // dependent launch: the first ring-full of weight tiles of my first unit goes out while the
      // kernel before this one is still running; the activations follow after griddep_wait
      int prefetched = 0;
      if (g.pdl) {
        const int u = blockIdx.x;
        if (u < num_units) {
          const int ks = u / num_tiles, tile = u % num_tiles;
          const int n0 = (tile % n_tiles) * BN;
          const int kb0 = ks * kb_per, kb1 = min(kb_total, kb0 + kb_per);
          for (int kb = kb0; kb < kb1 && prefetched < STAGES; ++kb, ++prefetched) {
            mbar_expect_tx(&full_bar[prefetched], STAGE_BYTES);      // the stages are all free at start
            load_b(smem + prefetched * STAGE_BYTES + A_BYTES, &full_bar[prefetched], kb * BK, n0);
          }
        }
      }
      griddep_wait();       // no-op unless launched as a dependent (decode step, captured training step)
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int ks = u / num_tiles;
        const int tile = u % num_tiles;
        const int m0 = (tile / n_tiles) * BM;
        const int n0 = (tile % n_tiles) * BN;
        const int kb0 = ks * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            *abort_flag = ST_TIMEOUT_EMPTY;
            atomicCAS(g.status, 0, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const bool b_done = prefetched > 0;       // this stage's B tile and byte count are already out
          if (b_done) --prefetched;
          else mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(sa + i * (BK * 128), &tmA, &full_bar[stage], m0 + i * 64, k0);
          }
          if (!b_done) load_b(sb, &full_bar[stage], k0, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16;
      constexpr uint32_t B_LBO = B_MN ? BK * 128 : 16;
      constexpr uint32_t A_KADV = A_MN ? UMMA_K * 128 : UMMA_K * 2;  // bytes per UMMA_K step
      constexpr uint32_t B_KADV = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++it) {
        const int ks = u / num_tiles;
        const int kb0 = ks * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        if (kb0 >= kb1) continue;
        const int ab = it & 1;
        if (!mbar_wait(&tempty_bar[ab], acc_phase[ab] ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_TMEM_EMPTY;
          atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[ab]);  // accumulator complete -> epilogue
        acc_phase[ab] ^= 1;
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue
    const int e = warp - 2;
    const int quad = warp & 3;           // TMEM lane quarter this warp may read
    const int part = e >> 2;             // which quarter of the BN columns
    constexpr int COLS_PER_WARP = BN / 4;
    uint8_t* my_stage = stage_out + e * 2048;
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    for (int u = blockIdx.x; u < num_units; u += gridDim.x, ++it) {
      const int ks = u / num_tiles;
      const int tile = u % num_tiles;
      const int kb0 = ks * kb_per;
      const int kb1 = min(kb_total, kb0 + kb_per);
      if (kb0 >= kb1) continue;
      const int ab = it & 1;
      const int m = (tile / n_tiles) * BM + quad * 32 + lane;
      const int nbase = (tile % n_tiles) * BN + part * COLS_PER_WARP;
      if (!mbar_wait(&tfull_bar[ab], acc_phase[ab], abort_flag)) {
        *abort_flag = ST_TIMEOUT_TMEM_FULL;
        atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      acc_phase[ab] ^= 1;
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ab * BN + part * COLS_PER_WARP;
      const int m0w = (tile / n_tiles) * BM + quad * 32;   // first row of this warp's block
      const bool row_ok = m < Meff;
      epilogue_drain<COLS_PER_WARP>(g, tmOut, tmAux, taddr, m, m0w, nbase, row_ok, my_stage, lane, ks == 0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[ab]);
    }
    if (lane == 0) tma_store_wait<0>();   // all of this warp's bulk stores have landed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes a 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (instruction shape 256 x 256 x 16).  CTA r of the pair stages rows
// [r*128, r*128+128) of the A tile and columns [r*128, r*128+128) of the B tile in its own shared
// memory (32 KB per stage instead of 48 KB, so the ring is five stages deep and each B byte is
// fetched by one SM instead of two) and owns accumulator rows [r*128, r*128+128) in its own TMEM.
// Only the leader (rank 0) issues MMAs.  Barrier protocol:
//   full[s]    leader only, 1 arrival (leader producer's expect_tx) + the bytes of both CTAs' loads
//   empty[s]   one per CTA, 1 arrival: the leader commits to its own and to the partner's
//   tfull[b]   one per CTA, 1 arrival: committed by the leader to both
//   tempty[b]  leader only, 2 x NUM_EPI_WARPS arrivals: the epilogue warps of both CTAs
// Loads are plain unicast TMA loads whose completion is counted on the leader's barrier.

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                              const __grid_constant__ CUtensorMap tmB,
                              const __grid_constant__ CUtensorMap tmOut,
                              const __grid_constant__ CUtensorMap tmAux, const GemmArgs g) {
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
  uint64_t* aux_bar = bars + 2 * STAGES + 5;      // one per epilogue warp: its staged aux tile
  static_assert((2 * STAGES + 5 + NUM_EPI_WARPS) * 8 <= 256, "barrier block outgrew its 256 bytes");

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
    for (int i = 0; i < NUM_EPI_WARPS; ++i) mbar_init(&aux_bar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmOut);
    if (g.ep.act == 1 || g.aux_tma) tma_prefetch_desc(&tmAux);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers are initialised before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // link of a programmatic chain (captured training step): the set-up above may have run while the
  // kernel before this one was draining; loads, the epilogue's reads and all stores come after
  if (threadIdx.x == 0) griddep_launch_dependents();
  griddep_wait();

  const int m_tiles = (g.M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = (g.N + BN - 1) / BN;
  const int kb_total = (g.K + BK - 1) / BK;
  const int kb_per = (kb_total + g.k_splits - 1) / g.k_splits;
  const int num_tiles = m_tiles * n_tiles;
  const int num_units = num_tiles * g.k_splits;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        const int ks = u / num_tiles;
        const int tile = u % num_tiles;
        const int m0 = (tile / n_tiles) * (2 * BM) + rank * BM;
        const int n0 = (tile % n_tiles) * BN + rank * HALF_N;
        const int kb0 = ks * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
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
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d_pair(sa + i * (BK * 128), &tmA, fb, m0 + i * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmB, fb, k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < HALF_N / 64; ++i)
              tma_load_2d_pair(sb + i * (BK * 128), &tmB, fb, n0 + i * 64, k0);
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
      for (int u = pair_id; u < num_units && ok; u += num_pairs, ++it) {
        const int ks = u / num_tiles;
        const int kb0 = ks * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        if (kb0 >= kb1) continue;
        const int ab = it & 1;
        if (!mbar_wait(&tempty_bar[ab], acc_phase[ab] ^ 1, abort_flag)) {
          *abort_flag = ST_TIMEOUT_TMEM_EMPTY;
          atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(mapa_shared(eb, 0));   // frees this stage in both CTAs
          umma_commit_pair(mapa_shared(eb, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t tb = smem_u32(&tfull_bar[ab]);
        umma_commit_pair(mapa_shared(tb, 0));     // accumulator complete -> both epilogues
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
    // GELU backward (act == 2): the warp's 32 x 64 tile of aux values is fetched by TMA into its
    // staging tile one unit ahead (right after the store of the unit before has read the tile), so
    // the loads that the epilogue math depends on are in flight while the accumulator is still
    // being computed instead of being issued, row by row, once it is ready.
    static_assert(COLS_PER_WARP == 64, "the staged aux tile is one 64-column store group");
    const bool stage_aux = g.aux_tma != 0;
    uint32_t aux_phase = 0;
    auto fetch_aux = [&](int u) {          // lane 0; the staging tile must be free
      if (u >= num_units) return;
      const int tile = u % num_tiles;
      const int m0w = (tile / n_tiles) * (2 * BM) + rank * BM + quad * 32;
      const int nbase = (tile % n_tiles) * BN + part * COLS_PER_WARP;
      if (m0w >= g.M || nbase >= g.N) return;       // the same test skips the drain below
      mbar_expect_tx(&aux_bar[e], 32 * 128);
      tma_load_2d(my_stage, &tmAux, &aux_bar[e], nbase, m0w);
    };
    if (stage_aux && lane == 0) fetch_aux(pair_id);
    int it = 0;
    for (int u = pair_id; u < num_units; u += num_pairs, ++it) {
      const int ks = u / num_tiles;
      const int tile = u % num_tiles;
      const int kb0 = ks * kb_per;
      const int kb1 = min(kb_total, kb0 + kb_per);
      if (kb0 >= kb1) continue;
      const int ab = it & 1;
      const int m0w = (tile / n_tiles) * (2 * BM) + rank * BM + quad * 32;
      const int m = m0w + lane;
      const int nbase = (tile % n_tiles) * BN + part * COLS_PER_WARP;
      if (!mbar_wait(&tfull_bar[ab], acc_phase[ab], abort_flag)) {
        *abort_flag = ST_TIMEOUT_TMEM_FULL;
        atomicCAS(g.status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      acc_phase[ab] ^= 1;
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ab * BN + part * COLS_PER_WARP;
      const bool staged = stage_aux && m0w < g.M && nbase < g.N;
      if (staged) {
        if (!mbar_wait(&aux_bar[e], aux_phase, abort_flag)) {
          *abort_flag = ST_TIMEOUT_FULL;
          atomicCAS(g.status, 0, ST_TIMEOUT_FULL);
          break;
        }
        aux_phase ^= 1;
      }
      // a warp whose 32 rows lie entirely past M has nothing to store (its accumulator rows came
      // from zero-filled loads); it still hands the buffer back
      if (m0w < g.M)
        epilogue_drain_wide<COLS_PER_WARP>(g, tmOut, tmAux, taddr, m, m0w, nbase, m < g.M, my_stage, lane,
                                           ks == 0, 0, staged);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[ab]), 0));
      if (stage_aux && lane == 0) {
        tma_store_wait_read<0>();           // the store just issued has read the staging tile
        fetch_aux(u + num_pairs);
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // nobody signals the partner's barriers or reads TMEM after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch_pair(const void* A, long long lda, const void* B, long long ldb, const GemmArgs& g,
                       int max_ctas, cudaStream_t stream) {
  constexpr int HALF_N = PAIR_BN / 2;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, g.M, g.K, lda, BM, BK, 2, true);
  else       rc = make_tmap_2d(&tmA, A, g.K, g.M, lda, BK, 64, 2, true);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, g.N, g.K, ldb, HALF_N, BK, 2, true);
  else       rc = make_tmap_2d(&tmB, B, g.K, g.N, ldb, BK, 64, 2, true);
  if (rc) return rc;
  CUtensorMap tmOut, tmAux;
  const AbGemmEpilogue& ep = g.ep;
  // store boxes of 32 rows with 128-byte rows (64-byte rows when two bf16 outputs share the tile)
  if (ep.out_fp32)       rc = make_tmap_2d_sw(&tmOut, ep.out, g.M, g.N, ep.ldo, 32, 32, 4, 128);
  else if (ep.act == 1)  rc = make_tmap_2d_sw(&tmOut, ep.out, g.M, g.N, ep.ldo, 32, 32, 2, 64);
  else                   rc = make_tmap_2d_sw(&tmOut, ep.out, g.M, g.N, ep.ldo, 32, 64, 2, 128);
  if (rc) return rc;
  GemmArgs ga = g;
  ga.aux_tma = 0;
  if (ep.act == 1) {
    rc = make_tmap_2d_sw(&tmAux, ep.aux, g.M, g.N, ep.ldaux, 32, 32, 2, 64);
    if (rc) return rc;
  } else if (ep.act == 2 && !ep.out_fp32 && !ep.accumulate && g.k_splits == 1 &&
             (reinterpret_cast<uintptr_t>(ep.aux) & 15) == 0 && (ep.ldaux * 2) % 16 == 0) {
    // the aux tiles travel by TMA in the geometry of the output tiles (see the kernel)
    rc = make_tmap_2d_sw(&tmAux, ep.aux, g.M, g.N, ep.ldaux, 32, 64, 2, 128);
    if (rc) return rc;
    ga.aux_tma = 1;
  } else {
    tmAux = tmOut;
  }
  constexpr int SMEM = 1024 + PAIR_STAGES * (BM * BK * 2 + HALF_N * BK * 2) +
                       NUM_EPI_WARPS * PAIR_WARP_STAGING + 256;
  auto kern = gemm_bf16_tcgen05_pair_kernel<A_MN, B_MN>;
  static PerDeviceOnce attr_set;
  if (attr_set.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set.mark_device();
  }
  const int m_tiles = (g.M + 2 * BM - 1) / (2 * BM), n_tiles = (g.N + PAIR_BN - 1) / PAIR_BN;
  const int units = m_tiles * n_tiles * g.k_splits;
  int pairs = max_ctas / 2;
  if (pairs > units) pairs = units;
  if (pairs < 1) pairs = 1;
  launch_chained(kern, dim3(2 * pairs), dim3(NUM_THREADS), SMEM, stream, tmA, tmB, tmOut, tmAux, ga);
  return static_cast<int>(cudaGetLastError());
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch(const void* A, long long lda, const void* B, long long ldb, const GemmArgs& g,
                  int max_ctas, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, g.M, g.K, lda, BM, BK, 2, true);
  else       rc = make_tmap_2d(&tmA, A, g.K, g.M, lda, BK, 64, 2, true);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, g.N, g.K, ldb, BN, BK, 2, true);
  else       rc = make_tmap_2d(&tmB, B, g.K, g.N, ldb, BK, 64, 2, true);
  if (rc) return rc;
  // output / pre-activation maps for the epilogue's TMA stores: boxes of 32 rows x 16 columns
  CUtensorMap tmOut, tmAux;
  const AbGemmEpilogue& ep = g.ep;
  if (ep.out_fp32) rc = make_tmap_2d_sw(&tmOut, ep.out, g.M, g.N, ep.ldo, 32, 16, 4, 64);
  else             rc = make_tmap_2d_sw(&tmOut, ep.out, g.M, g.N, ep.ldo, 32, 16, 2, 32);
  if (rc) return rc;
  if (ep.act == 1) {
    rc = make_tmap_2d_sw(&tmAux, ep.aux, g.M, g.N, ep.ldaux, 32, 16, 2, 32);
    if (rc) return rc;
  } else {
    tmAux = tmOut;
  }
  constexpr int SMEM = 1024 + STAGES * (BM * BK * 2 + BN * BK * 2) + NUM_EPI_WARPS * 2048 + 256;
  auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, A_MN, B_MN>;
  static PerDeviceOnce attr_set;
  if (attr_set.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set.mark_device();
  }
  const int m_tiles = (g.M + BM - 1) / BM, n_tiles = (g.N + BN - 1) / BN;
  const int units = m_tiles * n_tiles * g.k_splits;
  int grid = units < max_ctas ? units : max_ctas;
  if (grid < 1) grid = 1;
  if (g.pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmOut, tmAux, g));
  }
  launch_chained(kern, dim3(grid), dim3(NUM_THREADS), SMEM, stream, tmA, tmB, tmOut, tmAux, g);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ab

extern "C" int ab_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                            long long ldb, int M, int N, int K, const AbGemmEpilogue* ep,
                            int k_splits, int max_ctas, int* status, cudaStream_t stream) {
  using namespace ab;
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (lda & 7) || (ldb & 7) || !ep || !ep->out ||
      !status)
    return -1;
  if (k_splits < 1) k_splits = 1;
  if (k_splits > 1 && !(ep->out_fp32 && ep->accumulate)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(ep->out) | reinterpret_cast<uintptr_t>(ep->aux)) & 15)
    return -3;
  if ((ep->ldo * (ep->out_fp32 ? 4 : 2)) & 15) return -4;   // TMA row pitch: multiple of 16 bytes
  if (ep->act == 1 && (ep->ldaux & 7)) return -4;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K; g.k_splits = k_splits; g.ep = *ep; g.status = status; g.salt = seed_salt_ptr(); g.aux_tma = 0;
  // programmatic dependent launch: single-CTA kernels only, never with device-side limits (those
  // are values of earlier kernels, read before any wait)
  g.pdl = (ep->pdl && !ep->m_limit && !ep->k_limit) ? 1 : 0;
  if (max_ctas <= 0) max_ctas = 148;
  // narrow tiles also for skinny problems (decode steps with a few hundred rows): twice the CTAs
  const bool narrow = (N <= 128) || (M <= 256);
  // A few hundred rows against a wide weight matrix (decode steps): the time goes into streaming
  // the weights, so the columns are cut into 64-wide tiles to put twice as many SMs on them.
  if (M <= 256 && N >= 1024 && k_splits == 1) {
    if (!a_mn && !b_mn) return launch<64, 8, false, false>(A, lda, B, ldb, g, max_ctas, stream);
    if (!a_mn && b_mn) return launch<64, 8, false, true>(A, lda, B, ldb, g, max_ctas, stream);
  }
  if (narrow) {
    if (!a_mn && !b_mn) return launch<128, 6, false, false>(A, lda, B, ldb, g, max_ctas, stream);
    if (!a_mn && b_mn) return launch<128, 6, false, true>(A, lda, B, ldb, g, max_ctas, stream);
    if (a_mn && !b_mn) return launch<128, 6, true, false>(A, lda, B, ldb, g, max_ctas, stream);
    return launch<128, 6, true, true>(A, lda, B, ldb, g, max_ctas, stream);
  }
  // CTA pairs for the large shapes; the single-CTA kernel keeps the device-sized problems
  // (m_limit / k_limit) and anything a caller pins with AB_GEMM_NO_PAIR=1 in the environment
  static const bool no_pair = [] {
    const char* v = getenv("AB_GEMM_NO_PAIR");
    return v && v[0] == '1';
  }();
  if (!no_pair && !ep->m_limit && !ep->k_limit && M >= 512 && N >= 256 && max_ctas >= 2) {
    if (!a_mn && !b_mn) return launch_pair<false, false>(A, lda, B, ldb, g, max_ctas, stream);
    if (!a_mn && b_mn) return launch_pair<false, true>(A, lda, B, ldb, g, max_ctas, stream);
    if (a_mn && !b_mn) return launch_pair<true, false>(A, lda, B, ldb, g, max_ctas, stream);
    return launch_pair<true, true>(A, lda, B, ldb, g, max_ctas, stream);
  }
  if (!a_mn && !b_mn) return launch<256, 4, false, false>(A, lda, B, ldb, g, max_ctas, stream);
  if (!a_mn && b_mn) return launch<256, 4, false, true>(A, lda, B, ldb, g, max_ctas, stream);
  if (a_mn && !b_mn) return launch<256, 4, true, false>(A, lda, B, ldb, g, max_ctas, stream);
  return launch<256, 4, true, true>(A, lda, B, ldb, g, max_ctas, stream);
}
