// LoRA decode/prefill delta: y[t, :] += scale[s] * B[s] * (A[s] * x[t, :]) for the adapter
// slot s = slots[t] of each token (tokens with slot < 0 are untouched).  One CTA per
// token: the rank-r intermediate (r <= 128) lives in shared memory, A and B rows are
// streamed with 16-byte loads.  A: [slots, r_max, K], B: [slots, M, r_max], bf16.
//
// Functional parity with pegainfer-kernels/csrc/lora_fused.cu:102-375 (slot-indexed fused
// decode delta); projections that share an input are separate launches on row ranges.
#include "api.h"
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) lora_delta_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ A,
                                                          const bf16* __restrict__ B, const float* __restrict__ scale,
                                                          const int* __restrict__ slots, bf16* __restrict__ y, long long ldy, int K, int M,
                                                          int r_max, int num_slots) {
  __shared__ float tvec[128];
  const int t = blockIdx.x;
  const int s = slots[t];
  if (s < 0 || s >= num_slots) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* xr = x + t * ldx;
  const bf16* As = A + (long long)s * r_max * K;
  for (int r = warp; r < r_max; r += 8) {
    const bf16x8* ar = reinterpret_cast<const bf16x8*>(As + (long long)r * K);
    const bf16x8* xv = reinterpret_cast<const bf16x8*>(xr);
    float acc = 0.f;
    for (int i = lane; i < K / 8; i += 32) {
      float a[8], b[8];
      unpack8(ar[i], a);
      unpack8(xv[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += a[j] * b[j];
    }
    acc = warp_sum(acc);
    if (lane == 0) tvec[r] = acc;
  }
  __syncthreads();
  const float sc = scale[s];
  const bf16* Bs = B + (long long)s * M * r_max;
  for (int m = threadIdx.x; m < M; m += 256) {
    const bf16* br = Bs + (long long)m * r_max;
    float acc = 0.f;
    for (int r = 0; r < r_max; r += 8) {
      float b[8];
      unpack8(*reinterpret_cast<const bf16x8*>(br + r), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += b[j] * tvec[r + j];
    }
    y[t * ldy + m] = __float2bfloat16(__bfloat162float(y[t * ldy + m]) + sc * acc);
  }
}

}  // namespace

extern "C" int pg_lora_delta(const void* x, long long ldx, const void* A, const void* B, const void* scale, const void* slots, void* y,
                             long long ldy, int tokens, int K, int M, int r_max, int num_slots, cudaStream_t stream) {
  PG_REQUIRE(K % 8 == 0 && r_max % 8 == 0 && r_max <= 128, "lora_delta: K %% 8, rank %% 8 and rank <= 128 required (K=%d, r=%d)", K, r_max);
  if (tokens == 0) return PG_OK;
  lora_delta_kernel<<<tokens, 256, 0, stream>>>((const bf16*)x, ldx, (const bf16*)A, (const bf16*)B, (const float*)scale, (const int*)slots, (bf16*)y, ldy,
                                               K, M, r_max, num_slots);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
