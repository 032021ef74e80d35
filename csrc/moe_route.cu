// Mixture-of-experts routing kernels.
//
//  * router_topk: one warp per token over f32 logits [T, E] (E <= 512).  softmax or
//    sigmoid scores, optional selection bias, optional group-limited routing (keep the
//    `topk_group` best of `n_group` groups, group score = sum of its two best biased
//    scores), k rounds of warp arg-max (ties -> lowest expert id), weights from the
//    un-biased scores, optional renormalisation, scaling.
//  * moe_align: stable counting sort of the routes that hit local experts ->
//    expert offsets, source token per sorted row, sorted row per route.
//  * moe_gather / moe_combine: permute token rows into expert order, and the weighted
//    sum of each token's expert outputs in fixed slot order (deterministic).
//
// Functional parity with pegainfer-kernels/csrc/kimi_k2/kimi_router.cu:20-97,
// csrc/deepseek_v2_lite/dsv2_lite_moe.cu:41-216, csrc/kimi_k2/kimi_experts.cu:41-345.
#include <float.h>

#include "api.h"
#include "common.cuh"
#include "route_sort.cuh"

namespace {

constexpr int MAXE_PER_LANE = 16;  // E <= 512

struct RouterParams {
  const float* logits;
  long long ld;
  const float* bias;
  int* ids;
  float* weights;
  int tokens, E, k, sigmoid, n_group, topk_group, norm;
  float scale;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

__global__ void __launch_bounds__(128) router_topk_kernel(const RouterParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= p.tokens) return;
  const float* row = p.logits + t * p.ld;
  float score[MAXE_PER_LANE], choice[MAXE_PER_LANE];
  // expert e lives at lane e % 32, slot e / 32
  float mx = -FLT_MAX;
#pragma unroll
  for (int s = 0; s < MAXE_PER_LANE; ++s) {
    const int e = s * 32 + lane;
    score[s] = e < p.E ? row[e] : -FLT_MAX;
    mx = fmaxf(mx, score[s]);
  }
  if (p.sigmoid) {
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) {
      const int e = s * 32 + lane;
      score[s] = e < p.E ? 1.f / (1.f + expf(-score[s])) : 0.f;
    }
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) {
      const int e = s * 32 + lane;
      score[s] = e < p.E ? expf(score[s] - mx) : 0.f;
      sum += score[s];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) score[s] *= inv;
  }
#pragma unroll
  for (int s = 0; s < MAXE_PER_LANE; ++s) {
    const int e = s * 32 + lane;
    choice[s] = e < p.E ? score[s] + (p.bias ? p.bias[e] : 0.f) : -FLT_MAX;
  }
  if (p.n_group > 1) {
    // group g = experts [g*gs, (g+1)*gs); score = sum of its two best choices
    const int gs = p.E / p.n_group;
    uint32_t keep = 0u;  // bit g set = group g survives (n_group <= 32)
    float gscore_mine = -FLT_MAX;  // lane g holds group g's score
    for (int g = 0; g < p.n_group; ++g) {
      float b1 = -FLT_MAX, b2 = -FLT_MAX;
#pragma unroll
      for (int s = 0; s < MAXE_PER_LANE; ++s) {
        const int e = s * 32 + lane;
        if (e < p.E && e / gs == g) {
          const float c = choice[s];
          if (c > b1) {
            b2 = b1;
            b1 = c;
          } else if (c > b2) {
            b2 = c;
          }
        }
      }
      // merge (b1, b2) pairs across the warp
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1;
        b2 = n2;
      }
      const float gsc = gs >= 2 ? b1 + b2 : b1;
      if (lane == g) gscore_mine = gsc;
    }
    for (int r = 0; r < p.topk_group; ++r) {
      float v = lane < p.n_group && !((keep >> lane) & 1u) ? gscore_mine : -FLT_MAX;
      int i = lane;
      warp_argmax(v, i);
      keep |= 1u << i;
    }
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) {
      const int e = s * 32 + lane;
      if (e < p.E && !((keep >> (e / gs)) & 1u)) choice[s] = -FLT_MAX;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int r = 0; r < p.k; ++r) {
    float v = -FLT_MAX;
    int i = 0x7fffffff;
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) {
      const int e = s * 32 + lane;
      if (e < p.E && (choice[s] > v)) {  // ascending e per lane keeps the lowest id on ties
        v = choice[s];
        i = e;
      }
    }
    warp_argmax(v, i);
    // owner lane reads its un-biased score and retires the expert
    float sc = 0.f;
#pragma unroll
    for (int s = 0; s < MAXE_PER_LANE; ++s) {
      if (s * 32 + lane == i) {
        sc = score[s];
        choice[s] = -FLT_MAX;
      }
    }
    sc = __shfl_sync(0xffffffffu, sc, i & 31);
    wsum += sc;
    if (lane == r) {
      my_w = sc;
      my_id = i;
    }
  }
  if (lane < p.k) {
    float w = my_w;
    if (p.norm) w = w / (wsum + 1e-20f);
    p.ids[(long long)t * p.k + lane] = my_id;
    p.weights[(long long)t * p.k + lane] = w * p.scale;
  }
}

// One CTA: stable counting sort of the routes by local expert (see route_sort.cuh).
__global__ void __launch_bounds__(ROUTE_SORT_THREADS) moe_align_kernel(const int* __restrict__ ids, int routes, int e0, int e_local, int* __restrict__ offsets,
                                                                        int* __restrict__ sorted_src, int* __restrict__ route_pos) {
  __shared__ RouteSortSmem sm;
  route_sort(
      sm, routes, e_local, offsets, [&](int i) { return ids[i] - e0; },
      [&](int i, int pos) {
        route_pos[i] = pos;  // route index = token * k + slot
        if (pos >= 0) sorted_src[pos] = i;
      });
}

__global__ void moe_gather_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ sorted_src, const int* __restrict__ offsets,
                                  int e_local, int k, bf16* __restrict__ out, int width) {
  const int row = blockIdx.x;
  if (row >= offsets[e_local]) return;
  const int tok = sorted_src[row] / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + tok * ldx);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)row * width);
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t, :] (+)= sum_j weights[t, j] * y[route_pos[t*k + j], :]   (f32 output)
__global__ void moe_combine_kernel(const bf16* __restrict__ y, long long ldy, const int* __restrict__ route_pos, const float* __restrict__ weights,
                                   int k, float* __restrict__ out, int width, int accumulate) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
    float acc[8];
    float* op = out + (long long)t * width + i * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = accumulate ? op[j] : 0.f;
    for (int s = 0; s < k; ++s) {
      const int pos = route_pos[t * k + s];
      if (pos < 0) continue;
      const float w = weights[t * k + s];
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(y + pos * ldy)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) op[j] = acc[j];
  }
}

}  // namespace

extern "C" int pg_router_topk(const void* logits, long long ld, const void* bias, void* ids, void* weights, int tokens, int E, int k, int sigmoid,
                              int n_group, int topk_group, int norm, float scale, cudaStream_t stream) {
  PG_REQUIRE(E <= 32 * MAXE_PER_LANE && k >= 1 && k <= 32 && k <= E, "router: E=%d (<= 512) / k=%d (<= 32) out of range", E, k);
  PG_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group, "router: bad group routing %d/%d", topk_group, n_group);
  if (tokens == 0) return PG_OK;
  RouterParams p;
  p.logits = (const float*)logits;
  p.ld = ld;
  p.bias = (const float*)bias;
  p.ids = (int*)ids;
  p.weights = (float*)weights;
  p.tokens = tokens;
  p.E = E;
  p.k = k;
  p.sigmoid = sigmoid;
  p.n_group = n_group;
  p.topk_group = topk_group;
  p.norm = norm;
  p.scale = scale;
  router_topk_kernel<<<(tokens + 3) / 4, 128, 0, stream>>>(p);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_moe_align(const void* ids, int routes, int e0, int e_local, void* offsets, void* sorted_src, void* route_pos, cudaStream_t stream) {
  PG_REQUIRE(e_local >= 1 && e_local <= 512, "moe_align: %d local experts not supported (<= 512)", e_local);
  moe_align_kernel<<<1, ROUTE_SORT_THREADS, 0, stream>>>((const int*)ids, routes, e0, e_local, (int*)offsets, (int*)sorted_src, (int*)route_pos);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_moe_gather(const void* x, long long ldx, const void* sorted_src, const void* offsets, int e_local, int k, void* out, int width,
                             int max_rows, cudaStream_t stream) {
  PG_REQUIRE(width % 8 == 0, "moe_gather: width must be a multiple of 8");
  if (max_rows == 0) return PG_OK;
  moe_gather_kernel<<<max_rows, 128, 0, stream>>>((const bf16*)x, ldx, (const int*)sorted_src, (const int*)offsets, e_local, k, (bf16*)out, width);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_moe_combine(const void* y, long long ldy, const void* route_pos, const void* weights, int tokens, int k, void* out, int width,
                              int accumulate, cudaStream_t stream) {
  PG_REQUIRE(width % 8 == 0, "moe_combine: width must be a multiple of 8");
  if (tokens == 0) return PG_OK;
  moe_combine_kernel<<<tokens, 128, 0, stream>>>((const bf16*)y, ldy, (const int*)route_pos, (const float*)weights, k, (float*)out, width, accumulate);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
