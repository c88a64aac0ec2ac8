// Declarations shared by the attention kernels (forward, two-kernel backward, fused backward).
#pragma once
#include "ptx.cuh"

namespace ab {

constexpr int AT_BM = 128;   // query rows per CTA
constexpr int AT_BN = 128;   // keys per inner tile
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int B, T, H, hd;
  float scale;              // 1/sqrt(hd)
  unsigned long long seed;
  unsigned int stream_id, thr16;
  __nv_bfloat16* out;       // [B*T, H*hd]
  float* lse;               // [B, H, T]
  uint32_t* drop_mask;      // [B, H, T, T/32] keep bits written by the forward pass, or null
  const unsigned long long* salt;   // seed_salt_ptr() at launch: folded into `seed` when not null
  int* status;
};

// byte offset of the 16-byte chunk holding columns [8*c16, 8*c16+8) of row r inside a
// 128-row x 64-column bf16 panel with 128-byte swizzle (what TMA SWIZZLE_128B writes)
// order-preserving float <-> int coding (so integer atomicMax orders floats)
__device__ __forceinline__ int ord_encode(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ord_decode(int i) {
  return __int_as_float(i ^ ((i >> 31) & 0x7fffffff));
}

__device__ __forceinline__ uint32_t sw128_chunk(int r, int c16) {
  return static_cast<uint32_t>(r * 128 + ((c16 ^ (r & 7)) << 4));
}

struct AttnBwdArgs {
  int B, T, H, hd;
  float scale;
  unsigned long long seed;
  unsigned int stream_id, thr16;
  const float* lse;          // [B,H,T]
  const float* delta;        // [B,H,T]
  __nv_bfloat16* dqkv;       // [B*T, 3*H*hd]
  const uint32_t* drop_mask; // [B,H,T,T/32] keep bits from the forward pass, or null (recompute)
  float* dq_acc;             // [B*T, H*hd] fp32 accumulator for the single-kernel backward, or null
  const unsigned long long* salt;   // as in AttnArgs
  int* status;
};

}  // namespace ab
