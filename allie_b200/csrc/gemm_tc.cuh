// Public C interface of the tcgen05 GEMM (see gemm_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {

// Epilogue description.  All pointers are device pointers; null = feature off.
//   v = acc                                  (fp32, from TMEM)
//   v += bias[n]
//   act == 1:  aux[m][n] = bf16(v); v = gelu_new(v)
//   act == 2:  v *= gelu_new'(aux[m][n])
//   act == 3:  v = gelu_new(v)            (no pre-activation kept: inference)
//   aux_grad:  act == 1 stores aux[m][n] = bf16(gelu_new'(v)) instead of bf16(v), and act == 2
//              multiplies by aux[m][n] as it is (forward and backward must agree on the flag)
//   resid != null:  v = resid[m][n] + dropout(v)   (dropout only when drop_thr16 > 0)
//   out_fp32 ? (accumulate ? out[m][n] += v (atomic) : out[m][n] = v) : out[m][n] = bf16(v)
struct AbGemmEpilogue {
  void* out;
  long long ldo;
  int out_fp32;
  int accumulate;
  const float* bias;
  int act;
  void* aux;
  long long ldaux;
  const float* resid;
  long long ldr;
  unsigned long long drop_seed;
  unsigned int drop_stream;
  unsigned int drop_thr16;
  float alpha;  // v *= alpha before everything else (1.0 = off)
  // optional device-side problem sizes (null = use the host M / K): the kernel computes only
  // rows [0, min(M, *m_limit)) and contracts only over [0, min(K, *k_limit)).  Lets a launch be
  // sized for a capacity while the actual count (e.g. tokens routed to an expert) lives on the GPU.
  const int* m_limit;
  const int* k_limit;
  // nonzero: launch as a programmatic dependent of the kernel before it in the stream (small-M
  // launches that take the single-CTA kernel only): set-up and the prefetch of the first weight
  // tiles overlap that kernel; `B` must not be something it writes.
  int pdl;
  int aux_grad;
};

// C[M,N] = A[M,K] * B[K,N] on the 5th-generation tensor cores.
//   a_mn == 0: A stored row-major [M][K] (K contiguous), lda = row stride in elements
//   a_mn == 1: A stored row-major [K][M] (M contiguous)
//   b_mn == 0: B stored row-major [N][K] (K contiguous)
//   b_mn == 1: B stored row-major [K][N] (N contiguous)
// Requirements: bf16 operands, 16-byte aligned bases, lda/ldb multiples of 8,
// N a multiple of 8.  k_splits > 1 requires out_fp32 && accumulate.
// `status` is a device int the kernel sets to a nonzero StatusCode when a
// bounded wait ran out; the function itself returns a cudaError_t / negative
// value for host-side argument errors.
int ab_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn, long long ldb,
                 int M, int N, int K, const AbGemmEpilogue* ep, int k_splits, int max_ctas,
                 int* status, cudaStream_t stream);
}
