// Token selection kernels over logits rows [rows, vocab] (bf16 or f32).
//
//  * argmax: split partial/finalize, ties resolve to the lowest index; writes int32
//    tokens straight into the caller's buffer (the next decode step's input under a
//    CUDA graph).
//  * sample: one thread-block cluster per row (sample_cluster_kernel, below); the one-CTA kernel
//    described here serves vocabularies too large for eight CTAs' shared memory.  Online softmax at the row's temperature, then the
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

// One step of a low-rank Markov head over block-drafted logits: row r scores token v with
// base[(r * block + step) * ld + v] + bias[r * ldb + v] (bias = w2 . w1[previous token]); the best
// token becomes the row's previous token for the next step and entry (r, step) of the drafts.
template <typename T>
__global__ void __launch_bounds__(256) markov_partial_kernel(const T* __restrict__ base, long long ld, int block, int step, const T* __restrict__ bias,
                                                              long long ldb, int vocab, ArgPair* __restrict__ partial, int tiles) {
  PG_PDL_ENTRY();
  __shared__ ArgPair red[32];
  const int row = blockIdx.y, tile = blockIdx.x;
  const T* r = base + ((long long)row * block + step) * ld;
  const T* b = bias + (long long)row * ldb;
  ArgPair best{-FLT_MAX, 0x7fffffff};
  const int end = min(vocab, (tile + 1) * ARG_TILE);
  for (int i = tile * ARG_TILE + threadIdx.x; i < end; i += 256) {
    float v = ldf(r, i) + ldf(b, i);
    if (v > best.v) best = ArgPair{v, i};
  }
  best = block_argmax(best, red);
  if (threadIdx.x == 0) partial[(long long)row * tiles + tile] = best;
}

__global__ void __launch_bounds__(128) markov_final_kernel(const ArgPair* __restrict__ partial, int tiles, int* __restrict__ next, int* __restrict__ drafts,
                                                            int block, int step) {
  PG_PDL_ENTRY();
  __shared__ ArgPair red[32];
  const int row = blockIdx.x;
  ArgPair best{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < tiles; i += 128) best = arg_better(best, partial[(long long)row * tiles + i]);
  best = block_argmax(best, red);
  if (threadIdx.x == 0) {
    next[row] = best.i;
    drafts[(long long)row * block + step] = best.i;
  }
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
  __syncthreads();  // every thread has read the owner before anyone may change it below
  if (owner == ST) {  // uniform across the CTA
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

// ---------------------------------------------------------------------------------
// Cluster sampler: one thread-block cluster per row.  Each CTA of the cluster reads its slice
// of the row ONCE into shared memory (as tempered f32 logits) and every later pass -- the
// normaliser, the four radix levels of the threshold search, the inverse-CDF walk -- runs out
// of shared memory, with the per-CTA partial results combined across the cluster through
// distributed shared memory.  Probability mass is carried as 2^-40 fixed point in 64-bit
// integers, so every sum is exact and independent of the order in which threads add to it:
// the same (logits, controls, uniform) always pick the same token, and the CDF target
// floor(u * total) is always strictly inside the kept mass (no rounding fallback).
// ---------------------------------------------------------------------------------
constexpr int SC_THREADS = 512;
constexpr int SC_MAX_CLUSTER = 8;
constexpr float SC_FX = 1099511627776.f;  // 2^40

__device__ __forceinline__ unsigned long long ld_dsmem_u64(uint32_t cluster_addr) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_dsmem_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}

struct ScShared {
  unsigned long long h_mass[2][256];  // per-CTA histogram of the level being searched (double buffered)
  uint32_t h_cnt[2][256];
  unsigned long long m_mass[256];     // histogram merged over the cluster (every CTA computes the same)
  uint32_t m_cnt[256];
  unsigned long long x_u64;           // this CTA's contribution to a cluster-wide sum
  float x_f32;                        // this CTA's contribution to a cluster-wide max
  uint32_t prefix, cnt_above;
  unsigned long long mass_above;
  unsigned long long warp_tot[SC_THREADS / 32];
  int owner;
};

template <typename T>
__global__ void __launch_bounds__(SC_THREADS) sample_cluster_kernel(const T* __restrict__ logits, long long ld, int vocab, int slice,
                                                                    const float* __restrict__ temperature, const int* __restrict__ top_k,
                                                                    const float* __restrict__ top_p, const float* __restrict__ min_p,
                                                                    const float* __restrict__ uniform, int* __restrict__ out, int csize) {
  PG_PDL_ENTRY();
  extern __shared__ __align__(16) uint8_t sc_raw[];
  ScShared& sh = *reinterpret_cast<ScShared*>(sc_raw);
  float* vals = reinterpret_cast<float*>(sc_raw + ((sizeof(ScShared) + 15) & ~size_t(15)));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t cr = csize > 1 ? cluster_ctarank() : 0u;
  const int row = blockIdx.x / csize;
  const T* r = logits + row * ld;
  const float inv_t = 1.f / fmaxf(temperature[row], 1e-6f);
  const int i0 = min(vocab, (int)cr * slice), i1 = min(vocab, i0 + slice);
  const int n = i1 - i0;
  const int n_pad = (n + SC_THREADS - 1) / SC_THREADS * SC_THREADS;
  __shared__ float red[32];

  // the slice, tempered, into shared memory; local max
  float m = -FLT_MAX;
  for (int i = tid; i < n; i += SC_THREADS) {
    const float s = ldf(r, (long long)i0 + i) * inv_t;
    vals[i] = s;
    m = fmaxf(m, s);
  }
  m = block_max_f(m, red);
  if (tid == 0) {
    sh.x_f32 = m;
    sh.prefix = 0u;
    sh.cnt_above = 0u;
    sh.mass_above = 0ull;
  }
  for (int b = tid; b < 256; b += SC_THREADS) {
    sh.h_cnt[0][b] = 0u;
    sh.h_mass[0][b] = 0ull;
  }
  if (csize > 1) cluster_sync_all(); else __syncthreads();
  if (csize > 1) {
    float mm = -FLT_MAX;
    for (int q = 0; q < csize; ++q) mm = fmaxf(mm, ld_dsmem_f32(dsmem_addr(smem_u32(&sh.x_f32), (uint32_t)q)));
    m = mm;
  }

  const int kk = top_k[row] > 0 ? min(top_k[row], vocab) : vocab;
  const float tp = top_p[row];
  const float mp = min_p[row];

  // From here on a token is represented by e = exp(s - max) in (0, 1]: the exponential is taken
  // once, when the first radix level walks the slice, and stored over the tempered logit.  e
  // orders the tokens exactly as s does, so the threshold search runs on the bits of e; the
  // first level's histogram masses also add up to the normaliser.
  unsigned long long p_lim = ~0ull;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    const int hb = level & 1;
    const uint32_t prefix = sh.prefix;
    for (int i = tid; i < n_pad; i += SC_THREADS) {
      uint32_t bin = 256u;
      unsigned long long fx = 0ull;
      if (i < n) {
        float e = vals[i];
        if (level == 0) {
          e = __expf(e - m);
          vals[i] = e;
        }
        const uint32_t key = __float_as_uint(e);  // e >= 0: the bit pattern is already order preserving
        if ((key & hi_mask) == prefix) {
          bin = (key >> shift) & 255u;
          fx = (unsigned long long)(e * SC_FX);
        }
      }
      if (!__any_sync(0xffffffffu, bin < 256u)) continue;  // below the first level most warps have no candidate left
      // one shared-memory atomic per distinct bin of the warp
      const uint32_t peers = __match_any_sync(0xffffffffu, bin);
      if (bin < 256u) {
        const uint32_t lo = __reduce_add_sync(peers, (uint32_t)(fx & 0xFFFFFull));
        const uint32_t hi = __reduce_add_sync(peers, (uint32_t)(fx >> 20));
        if (lane == __ffs(peers) - 1) {
          atomicAdd(&sh.h_cnt[hb][bin], (uint32_t)__popc(peers));
          atomicAdd(&sh.h_mass[hb][bin], ((unsigned long long)hi << 20) + (unsigned long long)lo);
        }
      }
    }
    if (csize > 1) cluster_sync_all(); else __syncthreads();
    for (int b = tid; b < 256; b += SC_THREADS) {
      // The other buffer is free now: peers read it (the previous level's merge) before they arrived
      // at the barrier above.  The next level adds into it after the __syncthreads below.
      sh.h_cnt[hb ^ 1][b] = 0u;
      sh.h_mass[hb ^ 1][b] = 0ull;
      uint32_t c = 0u;
      unsigned long long ms = 0ull;
      if (csize > 1) {
        for (int q = 0; q < csize; ++q) {
          c += ld_dsmem_u32(dsmem_addr(smem_u32(&sh.h_cnt[hb][b]), (uint32_t)q));
          ms += ld_dsmem_u64(dsmem_addr(smem_u32(&sh.h_mass[hb][b]), (uint32_t)q));
        }
      } else {
        c = sh.h_cnt[hb][b];
        ms = sh.h_mass[hb][b];
      }
      sh.m_cnt[b] = c;
      sh.m_mass[b] = ms;
    }
    __syncthreads();
    if (warp == 0) {
      // Warp-parallel threshold step.  Lane l owns bins 8l .. 8l+7.  Walking the bins from the top, a
      // bin is kept while (count above < k) and (mass above < top-p limit); both grow as the bin index
      // falls, so the chosen bin is the LOWEST non-empty bin that still satisfies them.
      uint32_t c8[8];
      unsigned long long m8[8];
      uint32_t csum = 0u;
      unsigned long long msum = 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        c8[j] = sh.m_cnt[lane * 8 + j];
        m8[j] = sh.m_mass[lane * 8 + j];
        csum += c8[j];
        msum += m8[j];
      }
      // totals of the lanes above this one (exclusive suffix sum)
      uint32_t c_hi = csum;
      unsigned long long m_hi = msum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t cu = __shfl_down_sync(0xffffffffu, c_hi, o);
        const unsigned long long mu = __shfl_down_sync(0xffffffffu, m_hi, o);
        if (lane + o < 32) {
          c_hi += cu;
          m_hi += mu;
        }
      }
      if (level == 0) {
        const unsigned long long z = __shfl_sync(0xffffffffu, m_hi, 0);  // exact, whatever order the threads added in
        if (lane == 0) sh.x_u64 = tp >= 1.f ? ~0ull : (unsigned long long)((double)tp * (double)z);
        __syncwarp();
      }
      const unsigned long long lim = sh.x_u64;
      uint32_t cnt = sh.cnt_above + (c_hi - csum);
      unsigned long long mass = sh.mass_above + (m_hi - msum);
      int chosen = 256;
      uint32_t c_cnt = 0u;
      unsigned long long c_mass = 0ull;
#pragma unroll
      for (int j = 7; j >= 0; --j) {
        if (c8[j] != 0u && cnt < (uint32_t)kk && mass < lim) {
          chosen = lane * 8 + j;
          c_cnt = cnt;
          c_mass = mass;
        }
        cnt += c8[j];
        mass += m8[j];
      }
      int best = chosen;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
      __syncwarp();
      if (best == 256) {  // cannot happen (the top element is always kept); keep the top bin
        if (lane == 31) {
          sh.prefix = prefix | (255u << shift);
        }
      } else if (chosen == best) {  // exactly one lane owns the chosen bin
        sh.prefix = prefix | ((uint32_t)best << shift);
        sh.cnt_above = c_cnt;
        sh.mass_above = c_mass;
      }
    }
    __syncthreads();
  }
  (void)p_lim;
  // min-p: e >= min_p (e is relative to the row maximum, whose e is 1)
  const uint32_t thr_key = max(sh.prefix, mp > 0.f ? __float_as_uint(fminf(mp, 1.f)) : 0u);
  __syncthreads();  // every thread has read the threshold before x_u64 is reused below

  // inverse CDF in vocabulary order over the kept set: a contiguous chunk per thread
  const int chunk = (n + SC_THREADS - 1) / SC_THREADS;
  const int c0 = min(n, tid * chunk), c1 = min(n, c0 + chunk);
  unsigned long long local = 0ull;
  for (int i = c0; i < c1; ++i) {
    const float e = vals[i];
    if (__float_as_uint(e) >= thr_key) local += (unsigned long long)(e * SC_FX);
  }
  unsigned long long incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) sh.warp_tot[warp] = incl;
  __syncthreads();
  unsigned long long warp_before = 0ull, cta_total = 0ull;
  for (int w = 0; w < SC_THREADS / 32; ++w) {
    const unsigned long long t = sh.warp_tot[w];
    if (w < warp) warp_before += t;
    cta_total += t;
  }
  const unsigned long long before = warp_before + incl - local;
  if (tid == 0) {
    sh.x_u64 = cta_total;
    sh.owner = -1;
  }
  // x_u64 held the top-p limit, which only this CTA's thread 0 read (every CTA computes its own copy)
  if (csize > 1) cluster_sync_all(); else __syncthreads();
  unsigned long long total = 0ull, cta_before = 0ull;
  for (int q = 0; q < csize; ++q) {
    const unsigned long long t = csize > 1 ? ld_dsmem_u64(dsmem_addr(smem_u32(&sh.x_u64), (uint32_t)q)) : sh.x_u64;
    if (q < (int)cr) cta_before += t;
    total += t;
  }
  // u < 1, so the target lies strictly inside [0, total)
  const float u = fminf(fmaxf(uniform[row], 0.f), 0.99999994f);
  unsigned long long target = (unsigned long long)((double)u * (double)total);
  if (target >= total) target = total - 1ull;
  const bool mine = total > 0ull && target >= cta_before && target < cta_before + cta_total;
  if (mine) {
    const unsigned long long tl = target - cta_before;
    if (local > 0ull && before <= tl && tl < before + local) {
      unsigned long long acc = before;
      int pick = -1;
      for (int i = c0; i < c1; ++i) {
        const float e = vals[i];
        if (__float_as_uint(e) >= thr_key) {
          acc += (unsigned long long)(e * SC_FX);
          pick = i;
          if (acc > tl) break;
        }
      }
      out[row] = i0 + pick;
    }
  }
  // a CTA must not exit while a peer may still read its shared memory
  if (csize > 1) cluster_sync_all();
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

extern "C" int pg_markov_step_argmax(const void* base, int is_f32, int rows, int block, int step, int vocab, long long ld, const void* bias, long long ldb,
                                    void* scratch, long long scratch_bytes, void* next, void* drafts, cudaStream_t stream) {
  if (rows == 0) return PG_OK;
  const int tiles = ceil_div(vocab, ARG_TILE);
  PG_REQUIRE(step >= 0 && step < block, "markov step: step outside the block");
  PG_REQUIRE(scratch_bytes >= pg_argmax_scratch_bytes(rows, vocab), "markov step: scratch too small");
  dim3 grid(tiles, rows);
  if (is_f32)
    PG_CUDA(launch_pdl(markov_partial_kernel<float>, dim3(grid), dim3(256), (size_t)(0), stream, (const float*)base, ld, block, step, (const float*)bias, ldb,
                       vocab, (ArgPair*)scratch, tiles));
  else
    PG_CUDA(launch_pdl(markov_partial_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), stream, (const bf16*)base, ld, block, step, (const bf16*)bias, ldb, vocab,
                       (ArgPair*)scratch, tiles));
  PG_LAUNCH_CHECK();
  PG_CUDA(launch_pdl(markov_final_kernel, dim3(rows), dim3(128), (size_t)(0), stream, (const ArgPair*)scratch, tiles, (int*)next, (int*)drafts, block, step));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

static int g_force_cluster = 0;
// Test hook: pin the cluster size of the cluster sampler (1, 2, 4 or 8; 0 = chosen from the vocabulary).
extern "C" void pg_sample_force_cluster(int c) { g_force_cluster = c; }

// Cluster size and slice length of the cluster sampler for a vocabulary, or 0 when the row does
// not fit the shared memory of eight CTAs (the one-CTA kernel serves those).
static int sampler_cluster_plan(int vocab, int max_smem, int* slice_out) {
  const int room = (max_smem - 2048 - (int)sizeof(ScShared) - 64) / 4;  // floats per CTA (2 KB left for static shared memory)
  int c = 1;
  while (c < SC_MAX_CLUSTER && (ceil_div(vocab, c) > 24 * 1024 || ceil_div(vocab, c) > room)) c *= 2;
  if (g_force_cluster > 0) c = g_force_cluster;
  const int slice = (ceil_div(vocab, c) + 3) & ~3;
  if (slice > room) return 0;
  *slice_out = slice;
  return c;
}

template <typename T>
static int launch_sample_cluster(const T* logits, long long ld, int rows, int vocab, int c, int slice, const float* temperature, const int* top_k,
                                 const float* top_p, const float* min_p, const float* uniform, int* out, cudaStream_t stream) {
  const size_t smem = ((sizeof(ScShared) + 15) & ~size_t(15)) + (size_t)slice * 4;
  static bool attr_done[2] = {false, false};
  const int which = sizeof(T) == 4 ? 1 : 0;
  if (!attr_done[which]) {
    int max_smem = 0, dev = 0;
    PG_CUDA(cudaGetDevice(&dev));
    PG_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    PG_CUDA(cudaFuncSetAttribute(sample_cluster_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem - 2048));
    attr_done[which] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(rows * c));
  cfg.blockDim = dim3(SC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (c > 1) {
    at[na].id = cudaLaunchAttributeClusterDimension;
    at[na].val.clusterDim.x = (unsigned)c;
    at[na].val.clusterDim.y = 1;
    at[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_enabled()) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = (unsigned)na;
  PG_CUDA(cudaLaunchKernelEx(&cfg, sample_cluster_kernel<T>, logits, ld, vocab, slice, temperature, top_k, top_p, min_p, uniform, out, c));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_sample(const void* logits, int is_f32, int rows, int vocab, long long ld, const void* temperature, const void* top_k,
                         const void* top_p, const void* min_p, const void* uniform, void* out, cudaStream_t stream) {
  if (rows == 0) return PG_OK;
  static int use_cluster = -1, max_smem = 0;
  if (use_cluster < 0) {
    const char* e = getenv("PEGAINFER_SAMPLER_CLUSTER");
    int dev = 0;
    PG_CUDA(cudaGetDevice(&dev));
    PG_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    use_cluster = (e && e[0] == '0') ? 0 : 1;
  }
  int slice = 0;
  const int c = use_cluster ? sampler_cluster_plan(vocab, max_smem, &slice) : 0;
  if (c > 0) {
    if (is_f32)
      return launch_sample_cluster<float>((const float*)logits, ld, rows, vocab, c, slice, (const float*)temperature, (const int*)top_k, (const float*)top_p,
                                          (const float*)min_p, (const float*)uniform, (int*)out, stream);
    return launch_sample_cluster<bf16>((const bf16*)logits, ld, rows, vocab, c, slice, (const float*)temperature, (const int*)top_k, (const float*)top_p,
                                       (const float*)min_p, (const float*)uniform, (int*)out, stream);
  }
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
