// Stable counting sort of expert routes inside one CTA (shared by the local MoE path and
// the expert-parallel receive path).
//
// Routes arrive as a flat list of local expert ids (anything outside [0, e_local) means
// "not for this rank").  The list is staged through shared memory in chunks; every warp
// owns a subset of the experts and walks a chunk 32 entries at a time, ranking matches with
// a ballot, so the order inside an expert is the route order (stable: the f32 summation
// order downstream never depends on scheduling) while the scan is 32-wide.
//
// Takes the place of the reference's per-layer host-side routing bookkeeping and of the
// align step of its Marlin MoE path (pegainfer-kernels/csrc/kimi_k2/kimi_marlin_wna16.cu
// callers; pegainfer-deepseek-v2-lite/src/runtime/moe.rs).
#pragma once
#include "common.cuh"

constexpr int ROUTE_SORT_CHUNK = 8192;
constexpr int ROUTE_SORT_THREADS = 512;

struct RouteSortSmem {
  int ids[ROUTE_SORT_CHUNK];
  int cnt[512];
  int start[513];
};

// `load(i)` returns the local expert id of flat entry i (0 <= i < n); `emit(i, pos)` is called
// once per entry with its position in the sorted order, or pos = -1 when the entry is not
// for a local expert.  Writes offsets[0..e_local].  All ROUTE_SORT_THREADS threads call this.
template <typename Load, typename Emit>
__device__ __forceinline__ void route_sort(RouteSortSmem& sm, int n, int e_local, int* __restrict__ offsets, Load load, Emit emit) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = ROUTE_SORT_THREADS / 32;
  for (int e = threadIdx.x; e < 512; e += ROUTE_SORT_THREADS) sm.cnt[e] = 0;
  __syncthreads();
  // pass 1: counts
  for (int base = 0; base < n; base += ROUTE_SORT_CHUNK) {
    const int m = min(ROUTE_SORT_CHUNK, n - base);
    for (int i = threadIdx.x; i < m; i += ROUTE_SORT_THREADS) sm.ids[i] = load(base + i);
    __syncthreads();
    for (int e = warp; e < e_local; e += nwarps) {
      int c = 0;
      for (int i = lane; i < m; i += 32) c += (sm.ids[i] == e);
      c = (int)warp_sum((float)c);  // exact: counts stay far below 2^24
      if (lane == 0) sm.cnt[e] += c;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < e_local; ++i) {
      sm.start[i] = acc;
      acc += sm.cnt[i];
    }
    sm.start[e_local] = acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= e_local; i += ROUTE_SORT_THREADS) offsets[i] = sm.start[i];
  // pass 2: positions (sm.start[e] becomes the running cursor of expert e)
  for (int base = 0; base < n; base += ROUTE_SORT_CHUNK) {
    const int m = min(ROUTE_SORT_CHUNK, n - base);
    __syncthreads();
    for (int i = threadIdx.x; i < m; i += ROUTE_SORT_THREADS) {
      const int id = load(base + i);
      sm.ids[i] = id;
      if (id < 0 || id >= e_local) emit(base + i, -1);
    }
    __syncthreads();
    for (int e = warp; e < e_local; e += nwarps) {
      int running = sm.start[e];
      for (int i0 = 0; i0 < m; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < m && sm.ids[i] == e;
        const uint32_t mask = __ballot_sync(0xffffffffu, hit);
        if (hit) emit(base + i, running + __popc(mask & ((1u << lane) - 1u)));
        running += __popc(mask);
      }
      __syncwarp();
      if (lane == 0) sm.start[e] = running;
    }
  }
}
