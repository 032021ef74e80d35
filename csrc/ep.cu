// Expert-parallel dispatch / combine over NVLink peer memory (no host collectives).
//
// Every rank owns E/world experts.  Per MoE layer ("site") and step:
//
//   ep_dispatch      (sender)   one CTA per local token: for each of its k routes, store
//                               the token row into the owner rank's receive slab at the
//                               fixed slot [src rank][route]; tell every rank which local
//                               expert (or none) each of this rank's routes wants; then the
//                               last CTA raises this rank's "dispatched" epoch on all ranks.
//   ep_align         (owner)    waits for every source's dispatched epoch, then stable-
//                               sorts the received routes by local expert (same counting
//                               sort as the local path) -> offsets / sorted_src / route_pos.
//   grouped GEMMs    (owner)    W13, SwiGLU, W2 (moe_gemm.cu); the W2 epilogue stores each
//                               output row straight into the source rank's combine buffer
//                               and its tail raises the "returned" epoch on all ranks.
//   ep_combine       (sender)   waits for every owner's returned epoch, sums its tokens'
//                               k expert rows in slot order with the routing weights
//                               (deterministic), and advances the site's epoch.
//
// Slots are fixed functions of (source rank, token, slot), so there are no atomics on
// the data path and results do not depend on arrival order.  Flags are monotonic epochs
// in device memory: nothing is reset between steps or CUDA-graph replays.  All waits
// are bounded and report through the status word.
//
// Takes the place of the reference's DeepEP shim (dispatch prologue / dispatch /
// copy-epilogue / combine / reduce-epilogue, pegainfer-kernels/csrc/deepep/
// deepep_shim_impl.cuh:148-470) and of ncclAllToAll-style baselines.
#include "api.h"
#include "common.cuh"
#include "route_sort.cuh"

namespace {

constexpr int MAX_RANKS = 8;
constexpr int FLAG_WORDS = 32;  // [0..7] dispatched epoch per source, [8..15] returned epoch per owner, [16] epoch, [17],[18] CTA counters

struct EpPeers {
  bf16* slab[MAX_RANKS];      // [world][cap][H] on every rank
  int* recv_ids[MAX_RANKS];   // [world][cap] on every rank
  uint32_t* flags[MAX_RANKS];
  int rank, world, site;
  unsigned long long wait_ns;
};

__device__ __forceinline__ bool wait_epochs(const uint32_t* flags, int n, uint32_t target, unsigned long long limit_ns, uint32_t* status,
                                            uint32_t site) {
  const uint64_t t0 = globaltimer_ns();
  for (int q = 0; q < n; ++q) {
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flags + q) - target) < 0) {
      if ((++spins & 15u) == 0u) {
        if (*((volatile uint32_t*)status) != PG_ST_OK) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
          atomicCAS(status, PG_ST_OK, PG_ST_TIMEOUT | (site << 8) | ((uint32_t)q << 16));
          return false;
        }
      }
    }
  }
  return true;
}

// grid = tokens (bucket size, padding tokens included), 128 threads
__global__ void __launch_bounds__(128) ep_dispatch_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ ids, int tokens,
                                                           int valid_tokens_ptr_unused, const int* __restrict__ valid_tokens, int k, int hidden,
                                                           int e_local, int cap, const EpPeers p) {
  const int t = blockIdx.x;
  uint32_t* myflags = p.flags[p.rank] + p.site * FLAG_WORDS;
  const uint32_t next = *((volatile uint32_t*)&myflags[16]) + 1u;
  const int n_valid = valid_tokens ? *valid_tokens : tokens;
  const bool live = t < n_valid;
  for (int j = 0; j < k; ++j) {
    const int route = t * k + j;
    const int e = live ? ids[route] : -1;
    const int owner = e >= 0 ? e / e_local : -1;
    // every rank learns what this route wants from it (-1 = nothing)
    if (threadIdx.x < p.world) {
      const int q = threadIdx.x;
      p.recv_ids[q][(long long)p.rank * cap + route] = (q == owner) ? e - owner * e_local : -1;
    }
    if (owner >= 0) {
      const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
      uint4* dst = reinterpret_cast<uint4*>(p.slab[owner] + ((long long)p.rank * cap + route) * hidden);
      for (int i = threadIdx.x; i < hidden / 8; i += 128) dst[i] = src[i];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(&myflags[17], 1u);
    if (old == gridDim.x - 1) {
      myflags[17] = 0u;
      for (int q = 0; q < p.world; ++q) st_release_sys(p.flags[q] + p.site * FLAG_WORDS + p.rank, next);
    }
  }
}

// One CTA: wait for all sources, then the same stable counting sort as moe_align over the
// live part of the receive table (`live` routes per source; entries beyond that are left
// over from larger steps and must not be read).  The table is written by peers, so it is
// read past L1 (ld.cg) while being staged into shared memory.
__global__ void __launch_bounds__(ROUTE_SORT_THREADS) ep_align_kernel(const int* __restrict__ recv_ids, int world, int cap, int live, int e_local,
                                                                       int* __restrict__ offsets, int* __restrict__ sorted_src,
                                                                       const uint32_t* __restrict__ flags, unsigned long long wait_ns, uint32_t* status) {
  __shared__ RouteSortSmem sm;
  if (threadIdx.x == 0) {
    const uint32_t target = *((volatile const uint32_t*)(flags + 16)) + 1u;
    wait_epochs(flags, world, target, wait_ns, status, 8u);
  }
  __syncthreads();
  route_sort(
      sm, world * live, e_local, offsets, [&](int i) { return __ldcg(recv_ids + (i / live) * cap + (i % live)); },
      [&](int i, int pos) {
        if (pos >= 0) sorted_src[pos] = (i / live) * cap + (i % live);
      });
}

// out[t] = sum_j w[t, j] * comb[t*k + j]; grid = tokens.  The last CTA advances the epoch.
__global__ void __launch_bounds__(128) ep_combine_kernel(const bf16* __restrict__ comb, const int* __restrict__ ids, const float* __restrict__ weights,
                                                          int k, float* __restrict__ out, int hidden, const int* __restrict__ valid_tokens,
                                                          uint32_t* __restrict__ flags, int world, unsigned long long wait_ns, uint32_t* status) {
  __shared__ uint32_t s_ok;
  const int t = blockIdx.x;
  const uint32_t next = *((volatile uint32_t*)&flags[16]) + 1u;
  if (threadIdx.x == 0) s_ok = wait_epochs(flags + 8, world, next, wait_ns, status, 9u) ? 1u : 0u;
  __syncthreads();
  const int n_valid = valid_tokens ? *valid_tokens : (int)gridDim.x;
  for (int i = threadIdx.x; i < hidden / 8; i += 128) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (t < n_valid && s_ok) {
      for (int s = 0; s < k; ++s) {
        if (ids[t * k + s] < 0) continue;
        const float w = weights[t * k + s];
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(comb + (long long)(t * k + s) * hidden) + i);
        float f[8];
        unpack8(*reinterpret_cast<const bf16x8*>(&raw), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
      }
    }
    float* op = out + (long long)t * hidden + i * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) op[j] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(&flags[18], 1u);
    if (old == gridDim.x - 1) {
      flags[18] = 0u;
      __threadfence();
      *((volatile uint32_t*)&flags[16]) = next;
    }
  }
}

}  // namespace

static void fill_peers(EpPeers& p, void* const* slab, void* const* recv_ids, void* const* flags, int rank, int world, int site,
                       unsigned long long wait_ns) {
  for (int q = 0; q < world; ++q) {
    p.slab[q] = (bf16*)slab[q];
    p.recv_ids[q] = (int*)recv_ids[q];
    p.flags[q] = (uint32_t*)flags[q];
  }
  p.rank = rank;
  p.world = world;
  p.site = site;
  p.wait_ns = wait_ns;
}

// x [tokens, hidden] local tokens, ids [tokens, k] global expert ids; `cap` = route slots per
// source rank in the slabs (>= tokens * k).  `valid_tokens` (device int, may be null) marks
// the live prefix of a padded bucket.
extern "C" int pg_ep_dispatch(const void* x, long long ldx, const void* ids, int tokens, const void* valid_tokens, int k, int hidden, int e_local,
                              int cap, void* const* slab, void* const* recv_ids, void* const* flags, int rank, int world, int site,
                              unsigned long long wait_ns, cudaStream_t stream) {
  PG_REQUIRE(world >= 1 && world <= MAX_RANKS && tokens * k <= cap && hidden % 8 == 0, "ep_dispatch: bad geometry (world %d, routes %d, cap %d)", world, tokens * k, cap);
  if (tokens == 0) return PG_OK;
  EpPeers p;
  fill_peers(p, slab, recv_ids, flags, rank, world, site, wait_ns);
  ep_dispatch_kernel<<<tokens, 128, 0, stream>>>((const bf16*)x, ldx, (const int*)ids, tokens, 0, (const int*)valid_tokens, k, hidden, e_local, cap, p);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_ep_align(const void* recv_ids, int world, int cap, int live, int e_local, void* offsets, void* sorted_src, const void* site_flags,
                           unsigned long long wait_ns, void* status, cudaStream_t stream) {
  PG_REQUIRE(e_local >= 1 && e_local <= 512 && live <= cap, "ep_align: bad geometry (%d local experts, live %d, cap %d)", e_local, live, cap);
  ep_align_kernel<<<1, ROUTE_SORT_THREADS, 0, stream>>>((const int*)recv_ids, world, cap, live, e_local, (int*)offsets, (int*)sorted_src, (const uint32_t*)site_flags,
                                         wait_ns, (uint32_t*)status);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_ep_combine(const void* comb, const void* ids, const void* weights, int tokens, int k, void* out, int hidden,
                             const void* valid_tokens, void* site_flags, int world, unsigned long long wait_ns, void* status, cudaStream_t stream) {
  if (tokens == 0) return PG_OK;
  ep_combine_kernel<<<tokens, 128, 0, stream>>>((const bf16*)comb, (const int*)ids, (const float*)weights, k, (float*)out, hidden,
                                               (const int*)valid_tokens, (uint32_t*)site_flags, world, wait_ns, (uint32_t*)status);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
