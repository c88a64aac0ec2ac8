// Public C interface of the grouped tcgen05 GEMM (gemm_grouped.cu): one persistent CTA-pair
// launch that runs the same projection for all local experts of a mixture-of-experts layer.
#pragma once
#include "gemm_tc.cuh"

extern "C" {

struct AbGroupedGemm {
  int groups;        // local experts (<= 64)
  int cap;           // rows reserved per group in the row-indexed operands (multiple of 256)
  // mode 1 (forward / input gradient):  C[g] = A[g] * B[g], A[g] = rows [g*cap, g*cap + rows[g]) of A
  //        ([groups*cap, K], K contiguous); B[g] = group g of B ([groups][K][N] when b_mn, else
  //        [groups][N][K]); C rows sit like A's.  Only tiles that hold live rows are computed.
  // mode 2 (weight gradient):  C[g] (+)= A[g]^T * B[g], A = [groups*cap, M], B = [groups*cap, N],
  //        contraction over the rows of group g rounded up to 128; C = [groups][M][N] fp32, accumulated.
  int mode;
  const int* rows;                 // [groups] live rows per group (device memory)
  // Optional arrival counters, one per 128 rows of A (mode 1) / of the contraction (mode 2): a
  // block of rows is read only once its counter has reached the number of live rows in it.  The
  // rows may be written by other GPUs (peer stores followed by a release increment).
  const unsigned int* tile_ready;
  // Optional scattering epilogue (mode 1, bf16 output): row i of the result does not go to `out`
  // but to row (ret[i] & 0xffffff) of the buffer of rank (ret[i] >> 24), `peers[rank]`, a bf16
  // matrix of N columns.  When the last CTA is done, phase `phase` of the flag arrays is released
  // to every rank with `epoch`.
  const int* ret;
  void* peers[8];
  void* flags[8];
  int phase;
  unsigned int epoch;
  int rank, world;
  unsigned int* ticket;            // device counter, zero between launches
};

// Shapes: mode 1: A [groups*cap, K], N output columns; mode 2: M = columns of A, N = columns of B.
// `ep` as for ab_gemm_bf16 (bias: [groups][N]; act / aux as usual with aux laid out like out;
// no residual, no split-K, no device-side limits other than `rows`).
int ab_gemm_grouped_bf16(const void* A, long long lda, const void* B, int b_mn, long long ldb, int M,
                         int N, int K, const AbGemmEpilogue* ep, const AbGroupedGemm* grp,
                         int max_ctas, int* status, cudaStream_t stream);
}
