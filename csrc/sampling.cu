// Token selection kernels over logits rows [rows, vocab] (bf16 or f32).
//
//  * argmax: split partial/finalize, ties resolve to the lowest index; writes int32
//    tokens straight into the caller's buffer (the next decode step's input under a
//    CUDA graph).
//  * sample: one CTA per row.  Online softmax at the row's temperature, then the
//    keep-set {top-k AND top-p AND min-p} is found as a threshold on the scaled logit
//    by a 4-level byte-radix descent carrying (count, mass) of everything above, and
//    the token is drawn by inverse CDF in vocabulary order from one uniform per row,
//    so a replay with the same uniform is bit-reproducible.
//  * logprob_topk: log-softmax of the picked token plus the k best alternatives.
//
// Functional parity with pegainfer-kernels/csrc/shared/argmax.cu:91-230,
// flashinfer_sampling.cu:69-149 (softmax -> top-k/top-p/min-p sampling) and
// logprob_topk.cu:13-123.
#include <float.h>

#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) {
  return p[i];
}

constexpr int ARG_TILE = 4096;

struct ArgPair {
  float v;
  int i;
};
__device__ __forceinline__ ArgPair arg_better(ArgPair a, ArgPair b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgPair block_argmax(ArgPair a, ArgPair* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = arg_better(a, b);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = a;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  ArgPair t = lane < nw ? red[lane] : ArgPair{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = arg_better(t, b);
  }
  return t;
}

template <typename T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(const T* __restrict__ logits, long long ld, int vocab, ArgPair* __restrict__ partial,
                                                              int tiles) {
  PG_PDL_ENTRY();
  __shared__ ArgPair red[32];
  const int row = blockIdx.y, tile = blockIdx.x;
  const T* r = logits + row * ld;
  ArgPair best{-FLT_MAX, 0x7fffffff};
  const int end = min(vocab, (tile + 1) * ARG_TILE);
  for (int i = tile * ARG_TILE + threadIdx.x; i < end; i += 256) {
    float v = ldf(r, i);
    if (v > best.v) best = ArgPair{v, i};  // ascending i per thread keeps the lowest index on ties
  }
  best = block_argmax(best, red);
  if (threadIdx.x == 0) partial[(long long)row * tiles + tile] = best;
}

__global__ void __launch_bounds__(128) argmax_final_kernel(const ArgPair* __restrict__ partial, int tiles, int* __restrict__ out) {
  PG_PDL_ENTRY();
  __shared__ ArgPair red[32];
  const int row = blockIdx.x;
  ArgPair best{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < tiles; i += 128) best = arg_better(best, partial[(long long)row * tiles + i]);
  best = block_argmax(best, red);
  if (threadIdx.x == 0) out[row] = best.i;
}

// order-preserving float -> uint
__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int ST = 1024;  // sampler threads

__device__ __forceinline__ float block_sum_f(float v, float* red) { return block_sum(v, red); }
__device__ __forceinline__ float block_max_f(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < (int)((blockDim.x + 31) >> 5) ? red[lane] : -FLT_MAX;
  return warp_max(t);
}

template <typename T>
__global__ void __launch_bounds__(ST) sample_kernel(const T* __restrict__ logits, long long ld, int vocab, const float* __restrict__ temperature,
                                                     const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                     const float* __restrict__ min_p, const float* __restrict__ uniform, int* __restrict__ out) {
  PG_PDL_ENTRY();
  __shared__ float red[32];
  __shared__ uint32_t h_cnt[256];
  __shared__ float h_mass[256];
  __shared__ uint32_t s_prefix, s_cnt_above;
  __shared__ float s_mass_above;
  __shared__ float s_scan[ST];
  __shared__ int s_owner;
  const int row = blockIdx.x;
  const T* r = logits + row * ld;
  const float inv_t = 1.f / fmaxf(temperature[row], 1e-6f);
  const int tid = threadIdx.x;

  // pass 1: max and normaliser of the tempered row
  float m = -FLT_MAX;
  for (int i = tid; i < vocab; i += ST) m = fmaxf(m, ldf(r, i) * inv_t);
  m = block_max_f(m, red);
  float z = 0.f;
  for (int i = tid; i < vocab; i += ST) z += __expf(ldf(r, i) * inv_t - m);
  z = block_sum_f(z, red);

  const int kk = top_k[row] > 0 ? min(top_k[row], vocab) : vocab;
  const float p_lim = top_p[row] >= 1.f ? FLT_MAX : top_p[row] * z;
  const float mp = min_p[row];
  const float minp_thr = mp > 0.f ? m + __logf(mp) : -FLT_MAX;

  // radix descent on the key of the scaled logit: find the smallest kept key
  if (tid == 0) {
    s_prefix = 0;
    s_cnt_above = 0;
    s_mass_above = 0.f;
  }
  __syncthreads();
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    if (tid < 256) {
      h_cnt[tid] = 0;
      h_mass[tid] = 0.f;
    }
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int i = tid; i < vocab; i += ST) {
      const float s = ldf(r, i) * inv_t;
      const uint32_t key = fkey(s);
      if ((key & hi_mask) == prefix) {
        const uint32_t b = (key >> shift) & 255u;
        atomicAdd(&h_cnt[b], 1u);
        atomicAdd(&h_mass[b], __expf(s - m));
      }
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t cnt = s_cnt_above;
      float mass = s_mass_above;
      int chosen = -1;
      uint32_t c_cnt = cnt;
      float c_mass = mass;
      for (int b = 255; b >= 0; --b) {
        if (h_cnt[b] == 0) continue;
        if (cnt < (uint32_t)kk && mass < p_lim) {
          chosen = b;
          c_cnt = cnt;
          c_mass = mass;
        } else {
          break;
        }
        cnt += h_cnt[b];
        mass += h_mass[b];
      }
      if (chosen < 0) chosen = 255;  // cannot happen: the top element is always kept
      s_prefix = prefix | ((uint32_t)chosen << shift);
      s_cnt_above = c_cnt;
      s_mass_above = c_mass;
    }
    __syncthreads();
  }
  const uint32_t thr_key = max(s_prefix, fkey(minp_thr));

  // inverse CDF in vocabulary order over the kept set: contiguous chunk per thread
  const int chunk = (vocab + ST - 1) / ST;
  const int c0 = min(vocab, tid * chunk), c1 = min(vocab, c0 + chunk);
  float local = 0.f;
  for (int i = c0; i < c1; ++i) {
    const float s = ldf(r, i) * inv_t;
    if (fkey(s) >= thr_key) local += __expf(s - m);
  }
  s_scan[tid] = local;
  __syncthreads();
  // inclusive scan (Hillis-Steele over 1024 entries)
  for (int o = 1; o < ST; o <<= 1) {
    float add = tid >= o ? s_scan[tid - o] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float total = s_scan[ST - 1];
  const float target = uniform[row] * total;
  if (tid == 0) s_owner = ST;
  __syncthreads();
  const float before = tid ? s_scan[tid - 1] : 0.f;
  if (local > 0.f && before <= target && target < s_scan[tid]) atomicMin(&s_owner, tid);
  __syncthreads();
  int owner = s_owner;
  if (owner == ST) {
    // rounding pushed the target past the end: the last thread holding mass owns it
    if (local > 0.f) atomicMax(&s_owner, tid + ST);
    __syncthreads();
    owner = s_owner - ST;
  }
  if (tid == owner) {
    float acc = before;
    int pick = -1, last_kept = -1;
    for (int i = c0; i < c1; ++i) {
      const float s = ldf(r, i) * inv_t;
      if (fkey(s) >= thr_key) {
        last_kept = i;
        acc += __expf(s - m);
        if (acc > target) {
          pick = i;
          break;
        }
      }
    }
    out[row] = pick >= 0 ? pick : last_kept;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) logprob_topk_kernel(const T* __restrict__ logits, long long ld, int vocab, const int* __restrict__ picked,
                                                            int k, float* __restrict__ chosen_lp, float* __restrict__ top_lp,
                                                            int* __restrict__ top_idx) {
  PG_PDL_ENTRY();
  __shared__ float red[32];
  __shared__ ArgPair ared[32];
  __shared__ int taken[32];
  const int row = blockIdx.x;
  const T* r = logits + row * ld;
  float m = -FLT_MAX;
  for (int i = threadIdx.x; i < vocab; i += 256) m = fmaxf(m, ldf(r, i));
  m = block_max_f(m, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += 256) z += expf(ldf(r, i) - m);
  z = block_sum_f(z, red);
  const float lse = m + logf(z);
  if (threadIdx.x == 0) {
    int p = picked[row];
    chosen_lp[row] = (p >= 0 && p < vocab) ? ldf(r, p) - lse : -INFINITY;
  }
  for (int round = 0; round < k; ++round) {
    ArgPair best{-FLT_MAX, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += 256) {
      bool skip = false;
      for (int q = 0; q < round; ++q) skip |= (taken[q] == i);
      if (skip) continue;
      float v = ldf(r, i);
      if (v > best.v) best = ArgPair{v, i};
    }
    best = block_argmax(best, ared);
    if (threadIdx.x == 0) {
      taken[round] = best.i;
      top_lp[(long long)row * k + round] = best.v - lse;
      top_idx[(long long)row * k + round] = best.i;
    }
    __syncthreads();
  }
}

}  // namespace

extern "C" long long pg_argmax_scratch_bytes(int rows, int vocab) { return (long long)rows * ceil_div(vocab, ARG_TILE) * (long long)sizeof(ArgPair); }

extern "C" int pg_argmax(const void* logits, int is_f32, int rows, int vocab, long long ld, void* scratch, long long scratch_bytes, void* out,
                         cudaStream_t stream) {
  if (rows == 0) return PG_OK;
  const int tiles = ceil_div(vocab, ARG_TILE);
  PG_REQUIRE(scratch_bytes >= pg_argmax_scratch_bytes(rows, vocab), "argmax: scratch too small");
  dim3 grid(tiles, rows);
  if (is_f32)
    PG_CUDA(launch_pdl(argmax_partial_kernel<float>, dim3(grid), dim3(256), (size_t)(0), stream, (const float*)logits, ld, vocab, (ArgPair*)scratch, tiles));
  else
    PG_CUDA(launch_pdl(argmax_partial_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), stream, (const bf16*)logits, ld, vocab, (ArgPair*)scratch, tiles));
  PG_LAUNCH_CHECK();
  PG_CUDA(launch_pdl(argmax_final_kernel, dim3(rows), dim3(128), (size_t)(0), stream, (const ArgPair*)scratch, tiles, (int*)out));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_sample(const void* logits, int is_f32, int rows, int vocab, long long ld, const void* temperature, const void* top_k,
                         const void* top_p, const void* min_p, const void* uniform, void* out, cudaStream_t stream) {
  if (rows == 0) return PG_OK;
  if (is_f32)
    PG_CUDA(launch_pdl(sample_kernel<float>, dim3(rows), dim3(ST), (size_t)(0), stream, (const float*)logits, ld, vocab, (const float*)temperature, (const int*)top_k, (const float*)top_p,
                                                  (const float*)min_p, (const float*)uniform, (int*)out));
  else
    PG_CUDA(launch_pdl(sample_kernel<bf16>, dim3(rows), dim3(ST), (size_t)(0), stream, (const bf16*)logits, ld, vocab, (const float*)temperature, (const int*)top_k, (const float*)top_p,
                                                 (const float*)min_p, (const float*)uniform, (int*)out));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_logprob_topk(const void* logits, int is_f32, int rows, int vocab, long long ld, const void* picked, int k, void* chosen_lp,
                               void* top_lp, void* top_idx, cudaStream_t stream) {
  PG_REQUIRE(k >= 0 && k <= 32, "logprob_topk: k=%d out of range [0, 32]", k);
  if (rows == 0) return PG_OK;
  if (is_f32)
    PG_CUDA(launch_pdl(logprob_topk_kernel<float>, dim3(rows), dim3(256), (size_t)(0), stream, (const float*)logits, ld, vocab, (const int*)picked, k, (float*)chosen_lp, (float*)top_lp,
                                                         (int*)top_idx));
  else
    PG_CUDA(launch_pdl(logprob_topk_kernel<bf16>, dim3(rows), dim3(256), (size_t)(0), stream, (const bf16*)logits, ld, vocab, (const int*)picked, k, (float*)chosen_lp, (float*)top_lp,
                                                        (int*)top_idx));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
