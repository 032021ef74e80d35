// LoRA decode/prefill delta: y[t, :] += scale[s] * B[s] * (A[s] * x[t, :]) for the adapter
// slot s = slots[t] of each token (tokens with slot < 0 are untouched).  Two kernels: the
// shrink (A x, one warp per token and rank row, into an f32 [tokens, r] scratch) and the
// expand (B times that, a block per token and 1024 output columns); A and B rows are
// streamed with 16-byte loads.  A: [slots, r_max, K], B: [slots, M, r_max], bf16.
//
// Functional parity with pegainfer-kernels/csrc/lora_fused.cu:102-375 (slot-indexed fused
// decode delta); projections that share an input are separate launches on row ranges.
#include "api.h"
#include "common.cuh"

namespace {

// Shrink: tvec[t, r] = A[s, r, :] . x[t, :] for the token's adapter s; one warp per (token, rank row), eight rank rows per
// block.  Tokens without an adapter are skipped by both kernels.
__global__ void __launch_bounds__(256) lora_shrink_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ A, const int* __restrict__ slots,
                                                           float* __restrict__ tvec, int K, int r_max, int num_slots) {
  const int t = blockIdx.x;
  const int s = slots[t];
  if (s < 0 || s >= num_slots) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.y * 8 + warp;
  if (r >= r_max) return;
  const bf16x8* ar = reinterpret_cast<const bf16x8*>(A + ((long long)s * r_max + r) * K);
  const bf16x8* xv = reinterpret_cast<const bf16x8*>(x + t * ldx);
  float acc = 0.f;
  // independent loads in flight: a dependent L2 round trip per 16-byte chunk, not the bytes, was the cost of this loop
#pragma unroll 8
  for (int i = lane; i < K / 8; i += 32) {
    float a[8], b[8];
    unpack8(ar[i], a);
    unpack8(xv[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += a[j] * b[j];
  }
  acc = warp_sum(acc);
  if (lane == 0) tvec[(long long)t * r_max + r] = acc;
}

// Expand: y[t, m] += scale[s] * B[s, m, :] . tvec[t, :]; a block takes 1024 output columns of one token (four per thread).
__global__ void __launch_bounds__(256) lora_expand_kernel(const float* __restrict__ tvec, const bf16* __restrict__ B, const float* __restrict__ scale,
                                                           const int* __restrict__ slots, bf16* __restrict__ y, long long ldy, int M, int r_max, int num_slots) {
  __shared__ float tv[128];
  const int t = blockIdx.x;
  const int s = slots[t];
  if (s < 0 || s >= num_slots) return;
  if (threadIdx.x < r_max) tv[threadIdx.x] = tvec[(long long)t * r_max + threadIdx.x];
  __syncthreads();
  const float sc = scale[s];
  const bf16* Bs = B + (long long)s * M * r_max;
  const int m0 = blockIdx.y * 1024;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + i * 256 + threadIdx.x;
    if (m >= M) break;
    const bf16* br = Bs + (long long)m * r_max;
    float acc = 0.f;
    for (int r = 0; r < r_max; r += 8) {
      float b[8];
      unpack8(*reinterpret_cast<const bf16x8*>(br + r), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += b[j] * tv[r + j];
    }
    y[t * ldy + m] = __float2bfloat16(__bfloat162float(y[t * ldy + m]) + sc * acc);
  }
}

// Up to three projections that read the same input (q / k / v, gate / up) in one shrink and one expand launch:
// blockIdx.z selects the projection.
struct LoraMulti {
  const bf16* A[3];
  const bf16* B[3];
  bf16* y[3];
  long long ldy[3];
  int M[3];
  int n;
};

__global__ void __launch_bounds__(256) lora_shrink_multi_kernel(const bf16* __restrict__ x, long long ldx, const LoraMulti p, const int* __restrict__ slots, float* __restrict__ tvec, int K,
                                                                 int r_max, int num_slots, int tokens) {
  const int t = blockIdx.x, z = blockIdx.z;
  const int s = slots[t];
  if (s < 0 || s >= num_slots) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.y * 8 + warp;
  if (r >= r_max) return;
  const bf16x8* ar = reinterpret_cast<const bf16x8*>(p.A[z] + ((long long)s * r_max + r) * K);
  const bf16x8* xv = reinterpret_cast<const bf16x8*>(x + t * ldx);
  float acc = 0.f;
#pragma unroll 8
  for (int i = lane; i < K / 8; i += 32) {
    float a[8], b[8];
    unpack8(ar[i], a);
    unpack8(xv[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += a[j] * b[j];
  }
  acc = warp_sum(acc);
  if (lane == 0) tvec[((long long)z * tokens + t) * r_max + r] = acc;
}

__global__ void __launch_bounds__(256) lora_expand_multi_kernel(const float* __restrict__ tvec, const LoraMulti p, const float* __restrict__ scale, const int* __restrict__ slots, int r_max,
                                                                 int num_slots, int tokens) {
  __shared__ float tv[128];
  const int t = blockIdx.x, z = blockIdx.z;
  const int s = slots[t];
  if (s < 0 || s >= num_slots) return;
  const int M = p.M[z];
  const int m0 = blockIdx.y * 1024;
  if (m0 >= M) return;
  if (threadIdx.x < r_max) tv[threadIdx.x] = tvec[((long long)z * tokens + t) * r_max + threadIdx.x];
  __syncthreads();
  const float sc = scale[s];
  const bf16* Bs = p.B[z] + (long long)s * M * r_max;
  bf16* y = p.y[z] + t * p.ldy[z];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + i * 256 + threadIdx.x;
    if (m >= M) break;
    const bf16* br = Bs + (long long)m * r_max;
    float acc = 0.f;
    for (int r = 0; r < r_max; r += 8) {
      float b[8];
      unpack8(*reinterpret_cast<const bf16x8*>(br + r), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += b[j] * tv[r + j];
    }
    y[m] = __float2bfloat16(__bfloat162float(y[m]) + sc * acc);
  }
}

}  // namespace

extern "C" int pg_lora_delta(const void* x, long long ldx, const void* A, const void* B, const void* scale, const void* slots, void* y,
                             long long ldy, int tokens, int K, int M, int r_max, int num_slots, void* tvec, cudaStream_t stream) {
  PG_REQUIRE(K % 8 == 0 && r_max % 8 == 0 && r_max <= 128, "lora_delta: K %% 8, rank %% 8 and rank <= 128 required (K=%d, r=%d)", K, r_max);
  PG_REQUIRE(tvec != nullptr, "lora_delta: the [tokens, rank] f32 scratch is required");
  if (tokens == 0) return PG_OK;
  lora_shrink_kernel<<<dim3((unsigned)tokens, (unsigned)(r_max / 8)), 256, 0, stream>>>((const bf16*)x, ldx, (const bf16*)A, (const int*)slots, (float*)tvec, K, r_max, num_slots);
  PG_LAUNCH_CHECK();
  lora_expand_kernel<<<dim3((unsigned)tokens, (unsigned)((M + 1023) / 1024)), 256, 0, stream>>>((const float*)tvec, (const bf16*)B, (const float*)scale, (const int*)slots,
                                                                                              (bf16*)y, ldy, M, r_max, num_slots);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// The same for n <= 3 projections that share the input x: A[i] [slots, r_max, K], B[i] [slots, M[i], r_max], y[i] rows of
// stride ldy[i]; tvec is an f32 scratch of n * tokens * r_max.
extern "C" int pg_lora_delta_multi(const void* x, long long ldx, int n, const void* const* A, const void* const* B, void* const* y, const long long* ldy, const int* M,
                                   const void* scale, const void* slots, int tokens, int K, int r_max, int num_slots, void* tvec, cudaStream_t stream) {
  PG_REQUIRE(n >= 1 && n <= 3, "lora_delta_multi: 1 to 3 projections (got %d)", n);
  PG_REQUIRE(K % 8 == 0 && r_max % 8 == 0 && r_max <= 128, "lora_delta_multi: K %% 8, rank %% 8 and rank <= 128 required (K=%d, r=%d)", K, r_max);
  PG_REQUIRE(tvec != nullptr, "lora_delta_multi: the f32 scratch is required");
  if (tokens == 0) return PG_OK;
  LoraMulti p;
  int max_m = 0;
  for (int i = 0; i < 3; ++i) {
    const int j = i < n ? i : 0;
    p.A[i] = (const bf16*)A[j];
    p.B[i] = (const bf16*)B[j];
    p.y[i] = (bf16*)y[j];
    p.ldy[i] = ldy[j];
    p.M[i] = M[j];
    if (i < n && M[i] > max_m) max_m = M[i];
  }
  p.n = n;
  lora_shrink_multi_kernel<<<dim3((unsigned)tokens, (unsigned)(r_max / 8), (unsigned)n), 256, 0, stream>>>((const bf16*)x, ldx, p, (const int*)slots, (float*)tvec, K, r_max, num_slots,
                                                                                                           tokens);
  PG_LAUNCH_CHECK();
  lora_expand_multi_kernel<<<dim3((unsigned)tokens, (unsigned)((max_m + 1023) / 1024), (unsigned)n), 256, 0, stream>>>((const float*)tvec, p, (const float*)scale, (const int*)slots, r_max,
                                                                                                                        num_slots, tokens);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
