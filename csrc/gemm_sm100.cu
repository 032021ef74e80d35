// bf16 GEMM  Y[T, M] = X[T, K] * W[M, K]^T  on tcgen05 tensor cores.
//
// The weight matrix is the UMMA "A" operand (128 rows of W per tile fill the MMA M
// dimension) and the token rows are the "B" operand (N = token tile, 16..256), so a
// decode step with a handful of tokens still issues full-width 128-row MMAs and simply
// streams W through shared memory once: the kernel is HBM-bound for small T and
// tensor-bound for large T with the same code.
//
//   warp 0      TMA producer: W tile [128 x 64] and X tile [bn x 64] per stage
//   warp 1      allocates TMEM, issues tcgen05.mma (one thread), commits to mbarriers
//   warps 2..5  epilogue: tcgen05.ld the f32 accumulator (one TMEM lane = one W row per
//               thread), convert, store; two accumulator buffers so the epilogue of one
//               tile overlaps the main loop of the next
//
// Persistent grid, static round-robin over work items (tile, k-split).  With k-splits,
// every split writes an f32 partial into a workspace and bumps a per-tile counter; the
// CTA that arrives last sums the partials in split order (deterministic) and writes the
// output, then re-arms the counter, so the workspace needs no clearing between launches.
//
// Takes the place of the reference's cuBLAS/cuBLASLt layer
// (pegainfer-kernels/csrc/shared/linear.cu:294-596).
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int MAX_STAGES = 12;

constexpr int MAX_RANKS = 8;
constexpr int FLAG_WORDS_PER_SITE = 32;  // [0..7] tiles-done epoch per rank, [8..15] rows-delivered epoch per rank,
                                         // [16] epoch, [17]/[18] local CTA counters of the two phases

// Tensor-parallel tail fused behind the GEMM tiles: the tile epilogues push their f32
// partials into the receive buffers of the reducing ranks (reduce-scatter by posted peer
// stores), then + residual, RMSNorm, all-gather of the normalised rows.
struct TpFuse {
  int enabled;
  int rank, world, site;
  float* part[MAX_RANKS];      // every rank's receive buffer [source rank][rows][hidden] f32 (peer mapped)
  bf16* xout[MAX_RANKS];       // every rank's normalised-activation buffer [T, hidden]
  uint32_t* flags[MAX_RANKS];  // every rank's flag block
  bf16* residual;              // local [T, hidden]; rows owned by this rank are read and updated
  long long ld_res;
  const bf16* norm_w;
  float eps;
  int offset;
  int one_shot;            // 1: every rank reduces all rows itself and keeps them local (no gather hop)
  long long part_offset;   // element offset of this call's partial buffer inside every rank's `part` (double buffering)
  unsigned long long wait_ns;
  unsigned long long* timing;  // optional: 8 globaltimer stamps per site written by CTA 0 (profiling)
};

// Consumer side: X rows arrive from peers; wait for every rank's rows-delivered epoch.
struct WaitSpec {
  const uint32_t* flags;  // local flag block of the producing site (nullptr = no wait)
  int world;
  unsigned long long wait_ns;
  unsigned long long* timing;  // optional: [6] wait start, [7] wait end of the producing site's slot
};

// Work folded into the GEMM so that the decode chain needs no separate row kernels.
//
// Deferred RMSNorm: a row-parallel projection (EPI_RESID_NORMW) adds the residual, stores the new
// residual h and the un-normalised product xw = h * norm_w, and leaves per-(weight tile, token)
// sums of squares in `out_ssp`; the GEMM that consumes xw multiplies every output element of token
// n by inv_rms[n] = rsqrt(sum_tiles ssp[tile][n] / H + eps) in its epilogue (a per-token scalar
// commutes with the matrix product).  No kernel ever needs a whole row at once, so there is no
// grid-wide dependency between the projection and the norm.
//
// EPI_SWIGLU: the weight rows are interleaved (gate_0, up_0, gate_1, up_1, ...); the epilogue
// writes bf16(silu(g)) * u for every pair: out[n][m / 2].
enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_RESID_NORMW = 2 };
struct FuseSpec {
  int epi;
  const float* in_ssp;  // consumer side: [T][in_ld] sums of squares of the input rows, in_parts valid per row (nullptr = input is already normalised)
  int in_ld;            // row pitch of in_ssp in floats (a multiple of 4: rows are read with 16-byte loads)
  int in_parts;
  int in_width;         // H of the normalised vector
  float in_eps;
  bf16* residual;       // EPI_RESID_NORMW: [T, M] read, updated in place
  long long ld_res;
  const bf16* norm_w;   // EPI_RESID_NORMW: weight of the norm that the consumer completes
  int norm_offset;      // (1 + w) form
  float* out_ssp;       // EPI_RESID_NORMW: [T][out_ld], entry [n][m_tile]
  int out_ld;
};

struct GemmParams {
  TpFuse tp;
  WaitSpec wait;
  FuseSpec fuse;
  bf16* y;
  float* y_f32;
  long long ldy;
  int M, T, K;
  int bn;
  int m_tiles, n_tiles, kblocks, splits;
  int rotate;   // 1: each weight-row tile starts its k walk at a different k-block (spreads the L2 reads of the shared token tiles)
  int cluster;  // > 1: the k-splits of one tile are the CTAs of one cluster and reduce through distributed shared memory
  int stages;
  uint32_t tmem_cols;
  float* ws;
  uint32_t* counters;
  uint32_t* status;
  unsigned long long* timing;  // optional profiling: 16 globaltimer stamps per CTA (nullptr = off)
  const uint8_t* pf_ptr;  // weights of the next GEMM in the stream: pulled into L2 while this kernel runs
  long long pf_bytes;
};

// Where a finished f32 output element goes.  Plain GEMM: the local output.  Tensor-parallel
// partial: pushed (posted peer stores, no round trip) into the receive buffer
// [source rank][row][hidden] of the rank(s) that reduce this row, so that the transfer of a
// tile overlaps the MMAs of the tiles still being computed and the reduction later reads
// local memory only.
__device__ __forceinline__ void store_out(const GemmParams& p, int n, int m, float v, const float* s_inv = nullptr, int n_local = 0) {
  if (s_inv) v *= s_inv[n_local];
  if (p.tp.enabled) {
    const TpFuse& tp = p.tp;
    if (tp.one_shot) {
      const size_t off = (size_t)tp.part_offset + ((size_t)tp.rank * p.T + n) * p.M + m;
#pragma unroll
      for (int q = 0; q < MAX_RANKS; ++q)
        if (q < tp.world) tp.part[q][off] = v;
    } else {
      const int rows_per = (p.T + tp.world - 1) / tp.world;
      const int q = n / rows_per;
      tp.part[q][(size_t)tp.part_offset + ((size_t)tp.rank * rows_per + (n - q * rows_per)) * p.M + m] = v;
    }
  } else if (p.y_f32) {
    p.y_f32[(size_t)n * p.ldy + m] = v;
  } else {
    p.y[(size_t)n * p.ldy + m] = __float2bfloat16(v);
  }
}

// Row reduction of the tensor-parallel tail: sum the partials that the `W` ranks pushed
// into this rank's receive buffer (source q at src_row + q * src_stride) in rank order, add
// the residual, store it back, return this thread's share of the sum of squares.  All loops
// are unrolled at compile time so that up to 16 row vectors are in flight per thread and
// everything stays in registers (dynamic indexing would spill `buf` to local memory and
// serialise the loads).
constexpr int TP_KEEP = 12;
template <int W>
__device__ __forceinline__ float tp_sum_rows(const float* src_row, size_t src_stride, bf16* res_row, int lo, int hi, int iters, uint2 (&keep)[TP_KEEP]) {
  constexpr int GRP = (16 / W) < 1 ? 1 : (16 / W) > TP_KEEP ? TP_KEEP : (16 / W);
  constexpr int NB = (TP_KEEP + GRP - 1) / GRP;
  float ss = 0.f;
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    if (b * GRP < iters) {
      float4 buf[GRP][W];
      uint2 res[GRP];
#pragma unroll
      for (int g = 0; g < GRP; ++g) {
        const int it = b * GRP + g;
        const int i = lo + (int)threadIdx.x + it * NUM_THREADS;
        const bool live = it < TP_KEEP && it < iters && i < hi;
#pragma unroll
        for (int q = 0; q < W; ++q)
          buf[g][q] = live ? __ldcg(reinterpret_cast<const float4*>(src_row + (size_t)q * src_stride) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        res[g] = live ? *(reinterpret_cast<const uint2*>(res_row) + i) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int g = 0; g < GRP; ++g) {
        const int it = b * GRP + g;
        const int i = lo + (int)threadIdx.x + it * NUM_THREADS;
        if (it < TP_KEEP && it < iters && i < hi) {
          float4 a = buf[g][0];
#pragma unroll
          for (int q = 1; q < W; ++q) {
            a.x += buf[g][q].x;
            a.y += buf[g][q].y;
            a.z += buf[g][q].z;
            a.w += buf[g][q].w;
          }
          const float2 ra = __bfloat1622float2(*reinterpret_cast<const bf162*>(&res[g].x)), rb = __bfloat1622float2(*reinterpret_cast<const bf162*>(&res[g].y));
          const bf162 n0 = __floats2bfloat162_rn(a.x + ra.x, a.y + ra.y), n1 = __floats2bfloat162_rn(a.z + rb.x, a.w + rb.y);
          uint2 packed;
          packed.x = *reinterpret_cast<const uint32_t*>(&n0);
          packed.y = *reinterpret_cast<const uint32_t*>(&n1);
          *(reinterpret_cast<uint2*>(res_row) + i) = packed;
          if (it < TP_KEEP) keep[it] = packed;
          const float2 f0 = __bfloat1622float2(n0), f1 = __bfloat1622float2(n1);
          ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
        }
      }
    }
  }
  return ss;
}

// Four consecutive output features m..m+3 of token row n (the vector form of store_out).
// Returns this thread's contribution to the row's sum of squares (EPI_RESID_NORMW, else 0).
template <int EPI = EPI_PLAIN>
__device__ __forceinline__ float store_out4(const GemmParams& p, int n, int m, float4 v, const float* s_inv = nullptr, int n_local = 0,
                                            bool have_pre = false, uint2 pre_res = make_uint2(0u, 0u), uint2 pre_w = make_uint2(0u, 0u)) {
  if (s_inv) {
    const float sc = s_inv[n_local];
    v.x *= sc, v.y *= sc, v.z *= sc, v.w *= sc;
  }
  if (EPI == EPI_SWIGLU) {
    // rows (m, m+1) = (gate, up) of feature m / 2, rows (m+2, m+3) of the next one
    if (m + 3 < p.M) {
      const float g0 = bf16_round(v.x), u0 = bf16_round(v.y), g1 = bf16_round(v.z), u1 = bf16_round(v.w);
      const bf162 o = __floats2bfloat162_rn(bf16_round(g0 / (1.f + __expf(-g0))) * u0, bf16_round(g1 / (1.f + __expf(-g1))) * u1);
      *reinterpret_cast<bf162*>(p.y + (size_t)n * p.ldy + (m >> 1)) = o;
    }
    return 0.f;
  }
  if (EPI == EPI_RESID_NORMW) {
    if (m + 3 >= p.M) return 0.f;
    bf16* rr = p.fuse.residual + (size_t)n * p.fuse.ld_res + m;
    const uint2 rv = have_pre ? pre_res : *reinterpret_cast<const uint2*>(rr);
    const float2 r0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&rv.x)), r1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&rv.y));
    const bf162 h0 = __floats2bfloat162_rn(v.x + r0.x, v.y + r0.y), h1 = __floats2bfloat162_rn(v.z + r1.x, v.w + r1.y);
    uint2 hp;
    hp.x = *reinterpret_cast<const uint32_t*>(&h0);
    hp.y = *reinterpret_cast<const uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(rr) = hp;
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);  // the rounded sum is what gets normalised
    const uint2 wv = have_pre ? pre_w : *reinterpret_cast<const uint2*>(p.fuse.norm_w + m);
    float2 w0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&wv.x)), w1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&wv.y));
    if (p.fuse.norm_offset) w0.x += 1.f, w0.y += 1.f, w1.x += 1.f, w1.y += 1.f;
    const bf162 x0 = __floats2bfloat162_rn(f0.x * w0.x, f0.y * w0.y), x1 = __floats2bfloat162_rn(f1.x * w1.x, f1.y * w1.y);
    uint2 xp;
    xp.x = *reinterpret_cast<const uint32_t*>(&x0);
    xp.y = *reinterpret_cast<const uint32_t*>(&x1);
    *reinterpret_cast<uint2*>(p.y + (size_t)n * p.ldy + m) = xp;
    return f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
  }
  const bool vec = (p.M & 3) == 0 && m + 3 < p.M;
  if (!vec) {
    const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (m + i < p.M) store_out(p, n, m + i, f[i]);
    return 0.f;
  }
  if (p.tp.enabled) {
    const TpFuse& tp = p.tp;
    if (tp.one_shot) {
      const size_t off = (size_t)tp.part_offset + ((size_t)tp.rank * p.T + n) * p.M + m;
#pragma unroll
      for (int q = 0; q < MAX_RANKS; ++q)
        if (q < tp.world) *reinterpret_cast<float4*>(tp.part[q] + off) = v;
    } else {
      const int rows_per = (p.T + tp.world - 1) / tp.world;
      const int q = n / rows_per;
      *reinterpret_cast<float4*>(tp.part[q] + (size_t)tp.part_offset + ((size_t)tp.rank * rows_per + (n - q * rows_per)) * p.M + m) = v;
    }
  } else if (p.y_f32) {
    if ((p.ldy & 3) == 0)
      *reinterpret_cast<float4*>(p.y_f32 + (size_t)n * p.ldy + m) = v;
    else {
      float* o = p.y_f32 + (size_t)n * p.ldy + m;
      o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
    }
  } else {
    const bf162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    bf16* o = p.y + (size_t)n * p.ldy + m;
    if ((p.ldy & 3) == 0) {
      uint2 pk;
      pk.x = *reinterpret_cast<const uint32_t*>(&lo);
      pk.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(o) = pk;
    } else {
      o[0] = lo.x, o[1] = lo.y, o[2] = hi.x, o[3] = hi.y;
    }
  }
  return 0.f;
}

// Split-K reduction through distributed shared memory.  The k-splits of one output tile are
// the S CTAs of a cluster; the token columns are cut into S slices of `w` columns and CTA o
// reduces slice o.  Every CTA pushes slice o of its f32 partial into CTA o's shared memory
// (posted st.shared::cluster, slot [source CTA][column][128 rows]) and arrives on CTA o's
// mbarrier, so the reduction itself reads local shared memory only: this function sums the
// S slots in split order (deterministic) and stores the result.  A thread takes 4 rows of
// one column per pass, 4 columns per pass across the 128 epilogue threads.
// Residual values (4 bf16) of one token column of this thread's rows.
__device__ __forceinline__ uint2 load_resid(const GemmParams& p, int n, int m) {
  return (m + 3 < p.M) ? *reinterpret_cast<const uint2*>(p.fuse.residual + (size_t)n * p.fuse.ld_res + m) : make_uint2(0u, 0u);
}

// `first_res` / `norm_wv` (EPI_RESID_NORMW): the residual of this thread's first column and its norm
// weights, loaded by the caller while the main loop still ran; the residual of column i + 1 is loaded
// while column i is reduced, so no global load sits on the dependent path of the tail.
template <int EPI>
__device__ __forceinline__ void cluster_reduce_local(const GemmParams& p, const float* kred, int S, int w, uint32_t cr, int et, int n0, int m0, int m_tile,
                                                     const float* s_inv, uint2 first_res, uint2 norm_wv) {
  const int nmax = min(p.bn, p.T - n0);
  const int c_lo = (int)cr * w;
  const int ncols = min(nmax, c_lo + w) - c_lo;
  const int sub = et >> 5, r4 = (et & 31) * 4;
  uint2 cur = first_res;
  for (int j = sub; j < ncols; j += 4) {  // one warp = one token column across all 128 weight rows of the tile
    uint2 nxt = make_uint2(0u, 0u);
    if (EPI == EPI_RESID_NORMW && j + 4 < ncols) nxt = load_resid(p, n0 + c_lo + j + 4, m0 + r4);
    const float* src = kred + (size_t)j * BM + r4;
    float4 a = *reinterpret_cast<const float4*>(src);
#pragma unroll 4
    for (int q = 1; q < S; ++q) {
      const float4 b = *reinterpret_cast<const float4*>(src + (size_t)q * w * BM);
      a.x += b.x;
      a.y += b.y;
      a.z += b.z;
      a.w += b.w;
    }
    float ss = store_out4<EPI>(p, n0 + c_lo + j, m0 + r4, a, s_inv, c_lo + j, EPI == EPI_RESID_NORMW, cur, norm_wv);
    if (EPI == EPI_RESID_NORMW) {
      ss = warp_sum(ss);
      if ((et & 31) == 0) p.fuse.out_ssp[(size_t)(n0 + c_lo + j) * p.fuse.out_ld + m_tile] = ss;
      cur = nxt;
    }
  }
}

__device__ __forceinline__ bool named_bar_all(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(nthreads)
      : "memory");
  return r != 0;
}

// Wait until flags[0..n) >= target (monotonic epochs written by peers with release.sys).
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

// EPI / INV are compile-time so that each variant carries only its own epilogue: EPI is the fused
// epilogue (FuseSpec), INV says whether the input rows still owe their RMSNorm scale.
template <int EPI, bool INV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  const int stage_bytes = A_BYTES + p.bn * 128;
  float* kred = reinterpret_cast<float*>(tiles + p.stages * stage_bytes);  // [source CTA][slice column][128] f32, cluster mode only
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.stages * stage_bytes + (p.cluster > 1 ? (p.bn + 8) * BM * 4 : 0));
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* kfull = tempty + 2;  // every CTA of the cluster has pushed its slice into this CTA (4 warps x cluster arrivals)
  uint64_t* kfree = tempty + 3;  // every CTA of the cluster has reduced the previous item (its slots may be overwritten)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* last_flag = tmem_slot + 2;
  float* s_inv_buf = reinterpret_cast<float*>(tmem_slot + 4);  // [bn] inverse RMS of the input rows (deferred norm), epilogue threads only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* tstamp = p.timing ? p.timing + (size_t)blockIdx.x * 16 : nullptr;
  if (tstamp && threadIdx.x == 0) tstamp[0] = globaltimer_ns();

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    mbar_init(kfull, 4u * (uint32_t)p.cluster);
    mbar_init(kfree, 4u * (uint32_t)p.cluster);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if (p.cluster > 1) cluster_sync_all();  // peers' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: the prologue above, and the producer's first weight tiles
  // below, overlap the tail of the previous kernel in the stream; everything that reads or
  // writes activations, scratch or flags comes after pdl_wait().
  if (tstamp && threadIdx.x == 0) tstamp[1] = globaltimer_ns();
  if (threadIdx.x == 0) pdl_launch_dependents();
  else pdl_wait();
  if (p.tp.enabled && p.tp.timing && blockIdx.x == 0 && threadIdx.x == 0) p.tp.timing[p.tp.site * 8 + 0] = globaltimer_ns();

  const int total = p.m_tiles * p.n_tiles * p.splits;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t last_phase[MAX_STAGES];
      bool used[MAX_STAGES];
#pragma unroll
      for (int s = 0; s < MAX_STAGES; ++s) {
        used[s] = false;
        last_phase[s] = 0;
      }
      bool ok = true;
      bool x_ready = false;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int tile = item / p.splits, s = item - tile * p.splits;
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
        const int kb0 = (int)(((long long)p.kblocks * s) / p.splits);
        const int kb1 = (int)(((long long)p.kblocks * (s + 1)) / p.splits);
        int kb = kb0;
        // Every CTA of one k-split walks the same token tiles X[:, kb]; if they all walked them in
        // the same order, 32..192 SMs would ask L2 for the same few lines at the same moment and
        // the tiles would trickle in (measured: 8 KB per 0.26 us per SM).  Each weight-row tile
        // therefore starts its walk at a different k-block and wraps around (the order of the
        // partial sums depends on the tile's position only, never on the batch).
        const int nkb = kb1 - kb0;
        const int rot = p.rotate ? (m_tile * 3) % nkb : 0;
#define PG_KB(i) (kb0 + (((i) - kb0 + rot) % nkb))
        if (!x_ready) {
          // Weights never change, the token rows X come from the previous kernel (or, with the
          // all-gather fused into this GEMM, from peers): stream the first weight tiles, then
          // wait for the producer of X, then issue the X halves of those stages.
          const int pre = min(p.stages, kb1 - kb0);
          for (int i = 0; i < pre; ++i) {
            mbar_expect_tx(&full[i], (uint32_t)stage_bytes);
            tma_load_2d(tiles + i * stage_bytes, &tm_w, &full[i], PG_KB(kb0 + i) * BK, m_tile * BM, pol_w);
            used[i] = true;
            last_phase[i] = 0;
          }
          pdl_wait();
          if (tstamp) tstamp[2] = globaltimer_ns();
          if (p.wait.flags != nullptr) {
            // every rank's delivery epoch, then make the peer writes visible to the async proxy
            const uint32_t target = *((volatile const uint32_t*)(p.wait.flags + 16));
            if (p.wait.timing && blockIdx.x == 0) p.wait.timing[6] = globaltimer_ns();
            wait_epochs(p.wait.flags + 8, p.wait.world, target, p.wait.wait_ns, p.status, 2u);
            if (p.wait.timing && blockIdx.x == 0) p.wait.timing[7] = globaltimer_ns();
            fence_proxy_async_all();
          }
          x_ready = true;
          for (int i = 0; i < pre; ++i)
            tma_load_2d(tiles + i * stage_bytes + A_BYTES, &tm_x, &full[i], PG_KB(kb0 + i) * BK, n_tile * p.bn, pol_x);
          if (tstamp) tstamp[12] = globaltimer_ns();
          kb = kb0 + pre;
          stage = pre;
          if (stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        for (; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = tiles + stage * stage_bytes;
          mbar_expect_tx(&full[stage], (uint32_t)stage_bytes);
          tma_load_2d(a_dst, &tm_w, &full[stage], PG_KB(kb) * BK, m_tile * BM, pol_w);
          tma_load_2d(a_dst + A_BYTES, &tm_x, &full[stage], PG_KB(kb) * BK, n_tile * p.bn, pol_x);
          used[stage] = true;
          last_phase[stage] = phase;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (tstamp) tstamp[3] = globaltimer_ns();
      // All of this CTA's own loads are issued.  From here to the first load of the next GEMM
      // in the stream (epilogue, launch gap, the small kernel in between, the next prologue)
      // HBM would sit idle: pull a slice of the NEXT GEMM's weights into L2 meanwhile
      // (weights never change, so no ordering is needed; the prefetch is fire-and-forget).
      if (p.pf_bytes > 0) {
        constexpr long long CH = 16384;
        const long long nch = (p.pf_bytes + CH - 1) / CH;
        for (long long c = blockIdx.x; c < nch; c += gridDim.x) {
          const long long left = p.pf_bytes - c * CH;
          const uint32_t sz = (uint32_t)(left < CH ? left : CH) & ~15u;
          if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf_ptr + c * CH), "r"(sz) : "memory");
        }
      }
      // Drain: every bulk copy this thread issued must have landed before the CTA exits.
      for (int s = 0; s < p.stages; ++s) {
        if (!used[s]) continue;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&full[s], last_phase[s])) {
          if (globaltimer_ns() - t0 > PG_WAIT_LIMIT_NS) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(BM, (uint32_t)p.bn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int tile = item / p.splits, s = item - tile * p.splits;
        const int kb0 = (int)(((long long)p.kblocks * s) / p.splits);
        const int kb1 = (int)(((long long)p.kblocks * (s + 1)) / p.splits);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          if (tstamp && item == (int)blockIdx.x && kb == kb0) tstamp[4] = globaltimer_ns();
          if (tstamp && item == (int)blockIdx.x && kb == kb0 + 1) tstamp[13] = globaltimer_ns();
          if (tstamp && item == (int)blockIdx.x && kb == kb0 + 6) tstamp[14] = globaltimer_ns();
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16_ss(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (tstamp) tstamp[5] = globaltimer_ns();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int et = threadIdx.x - 64;  // 0..127 among epilogue threads
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t kphase = 0;
    const uint32_t cr = p.cluster > 1 ? cluster_ctarank() : 0u;
    const int kw = p.cluster > 1 ? (p.bn + p.cluster - 1) / p.cluster : p.bn;  // columns per slice
    bool cluster_arrived = false;
    const float* s_inv = INV ? s_inv_buf : nullptr;
    int inv_tile = -1;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      const int tile = item / p.splits, s = item - tile * p.splits;
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      if (INV && n_tile != inv_tile) {
        // inverse RMS of this token tile's input rows, from the producer's per-tile sums of squares
        // (fixed summation order); computed while the main loop runs
        if (inv_tile >= 0) named_bar_all(1, 128, true);  // nobody still reads the previous tile's values
        // one thread per token: the row's per-tile sums are contiguous, read with 16-byte loads that are
        // all in flight together, summed in ascending tile order
        for (int nl = et; nl < p.bn; nl += 128) {
          const int n = n_tile * p.bn + nl;
          float ss = 0.f;
          if (n < p.T) {
            const float4* src = reinterpret_cast<const float4*>(p.fuse.in_ssp + (size_t)n * p.fuse.in_ld);
            for (int q = 0; q < p.fuse.in_parts; q += 32) {
              float4 v[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) v[u] = (q + 4 * u < p.fuse.in_parts) ? __ldcg(src + (q >> 2) + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const int b = q + 4 * u;
                ss += (b < p.fuse.in_parts ? v[u].x : 0.f);
                ss += (b + 1 < p.fuse.in_parts ? v[u].y : 0.f);
                ss += (b + 2 < p.fuse.in_parts ? v[u].z : 0.f);
                ss += (b + 3 < p.fuse.in_parts ? v[u].w : 0.f);
              }
            }
          }
          s_inv_buf[nl] = rsqrtf(ss / (float)p.fuse.in_width + p.fuse.in_eps);
        }
        inv_tile = n_tile;
      }
      uint2 first_res = make_uint2(0u, 0u), norm_wv = make_uint2(0u, 0u);
      if (EPI == EPI_RESID_NORMW && p.cluster > 1) {
        // this thread's norm weights and the residual of its first column, fetched while the main loop runs
        const int mm = m_tile * BM + (et & 31) * 4, n_first = n_tile * p.bn + (int)cr * kw + (et >> 5);
        if (mm + 3 < p.M) norm_wv = *reinterpret_cast<const uint2*>(p.fuse.norm_w + mm);
        if (n_first < p.T) first_res = load_resid(p, n_first, mm);
      }
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag);
      // cluster mode: every owner must have reduced the previous item before its slots are overwritten
      if (p.cluster > 1) ok = mbar_wait_cluster(kfree, kphase ^ 1u, abort_flag) && ok;
      ok = named_bar_all(1, 128, ok);
      if (!ok) break;
      if (tstamp && et == 0) tstamp[6] = globaltimer_ns();
      tc_fence_after();
      const int m = m_tile * BM + r;
      const int n0 = n_tile * p.bn;
      const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * p.bn);
      float* ws_part = p.ws + ((size_t)(tile * p.splits + s) * p.bn) * BM + r;
      if (p.cluster > 1) {
        // push the partial: column c belongs to slice c / kw, i.e. to CTA c / kw of the cluster;
        // 32 accumulator columns per TMEM round trip, one running remote address per slice
        const uint32_t slot = smem_u32(kred) + (uint32_t)(((int)cr * kw) * BM + r) * 4u;  // this CTA's slot, same offset in every owner
        int owner = 0, jj = 0;
        uint32_t dst = dsmem_addr(slot, 0u);
        for (int c = 0; c < p.bn; c += 32) {
          uint32_t v[2][16];
          tmem_ld16(t_row + c, v[0]);
          if (c + 16 < p.bn) tmem_ld16(t_row + c + 16, v[1]);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (c + h * 16 < p.bn) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                st_dsmem_f32(dst, __uint_as_float(v[h][j]));
                dst += BM * 4u;
                if (++jj == kw) {
                  jj = 0;
                  ++owner;
                  dst = dsmem_addr(slot, (uint32_t)min(owner, p.cluster - 1));
                }
              }
            }
          }
        }
      } else {
        for (int c = 0; c < p.bn; c += 16) {
          uint32_t v[16];
          tmem_ld16(t_row + c, v);
          tmem_ld_wait();
          if (p.splits == 1) {
            if (m < p.M) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int n = n0 + c + j;
                if (n < p.T) store_out(p, n, m, __uint_as_float(v[j]), s_inv, c + j);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) ws_part[(size_t)(c + j) * BM] = __uint_as_float(v[j]);
          }
        }
      }
      // accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

      if (p.cluster > 1) {
        // every CTA has pushed its slices once all 4 x S warps have arrived on this CTA's barrier
        const uint32_t S = (uint32_t)p.cluster;
        const bool last_item = item + (int)gridDim.x >= total;
        __syncwarp();
        if ((uint32_t)lane < S) mbar_arrive_remote(dsmem_addr(smem_u32(kfull), (uint32_t)lane));
        if (last_item) {
          cluster_arrive_release();  // no further access to the peers' shared memory from this thread
          cluster_arrived = true;
        }
        if (tstamp && et == 0) tstamp[7] = globaltimer_ns();
        const bool full_ok = named_bar_all(1, 128, mbar_wait_cluster(kfull, kphase, abort_flag));
        if (tstamp && et == 0) tstamp[8] = globaltimer_ns();
        if (full_ok) cluster_reduce_local<EPI>(p, kred, (int)S, kw, cr, et, n0, m_tile * BM, m_tile, s_inv, first_res, norm_wv);
        if (tstamp && et == 0) tstamp[9] = globaltimer_ns();
        // this CTA's slots may be overwritten by the next item (also said on the abort path, so nobody waits in vain)
        if (!last_item) {
          __syncwarp();
          if ((uint32_t)lane < S) mbar_arrive_remote(dsmem_addr(smem_u32(kfree), (uint32_t)lane));
        }
        kphase ^= 1u;
        if (!full_ok) break;
      } else if (p.splits > 1) {
        __threadfence();
        named_bar_all(1, 128, true);
        if (et == 0) {
          const uint32_t old = atomicAdd(&p.counters[tile], 1u);
          *last_flag = (old == (uint32_t)(p.splits - 1)) ? 1u : 0u;
        }
        named_bar_all(1, 128, true);
        if (*last_flag) {
          __threadfence();
          const float* ws_tile = p.ws + ((size_t)tile * p.splits * p.bn) * BM + r;
          const int nmax = min(p.bn, p.T - n0);
          // 16 columns at a time, four splits' loads in flight together: the loop is
          // bound by L2 latency, so independent loads must not be serialised by stores
          for (int c = 0; c < nmax; c += 16) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            for (int q0 = 0; q0 < p.splits; q0 += 4) {
              float tmp[4][16];
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const bool live = q0 + qq < p.splits;
                const float* src = ws_tile + ((size_t)(live ? q0 + qq : q0) * p.bn + c) * BM;
#pragma unroll
                for (int j = 0; j < 16; ++j) tmp[qq][j] = live ? __ldcg(src + (size_t)j * BM) : 0.f;
              }
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += tmp[qq][j];
              }
            }
            if (m < p.M) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int n = c + j;
                if (n < nmax) store_out(p, n0 + n, m, acc[j], s_inv, n);
              }
            }
          }
          if (et == 0) p.counters[tile] = 0u;
        }
      }
    }
    if (p.cluster > 1 && !cluster_arrived) cluster_arrive_release();  // no items, or the loop ended early
  }
  // producer and MMA warps never touch the peers' shared memory
  if (p.cluster > 1 && warp < 2) cluster_arrive_release();

  tc_fence_before();
  __syncthreads();
  if (tstamp && threadIdx.x == 0) tstamp[10] = globaltimer_ns();
  // No CTA may leave while a peer can still push into its shared memory or arrive on its
  // barriers: every thread of the cluster has arrived once it is past its last remote access
  // (the epilogue threads right after pushing the last item), so this wait is normally over
  // by the time the local reduction has finished.
  if (p.cluster > 1) cluster_wait_acquire();
  if (tstamp && threadIdx.x == 0) tstamp[11] = globaltimer_ns();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (1u << 8));

  if (p.tp.enabled) {
    // ---- reduce-scatter + residual + RMSNorm + all-gather over peer memory ----
    const TpFuse& tp = p.tp;
    const int H = p.M;
    uint32_t* myflags = tp.flags[tp.rank] + tp.site * FLAG_WORDS_PER_SITE;
    // the epoch advances only after every CTA of this launch has finished its tail, so each CTA reads the same value here
    const uint32_t tp_epoch = *((volatile uint32_t*)&myflags[16]);
    const uint32_t next = tp_epoch + 1u;
    unsigned long long* tm = (tp.timing && blockIdx.x == 0 && threadIdx.x == 0) ? tp.timing + tp.site * 8 : nullptr;
    if (tm) tm[1] = globaltimer_ns();
    float* red = reinterpret_cast<float*>(tiles);       // pipeline smem is idle now
    uint32_t* s_ok = reinterpret_cast<uint32_t*>(tiles) + 64;
    // phase 1 done: the last CTA of this GPU tells every rank that all partial tiles are stored
    if (threadIdx.x == 0) {
      __threadfence_system();
      const uint32_t old = atomicAdd(&myflags[17], 1u);
      if (old == gridDim.x - 1) {
        myflags[17] = 0u;
        __threadfence_system();  // acquire side of the counter: every CTA's pushed tiles precede the signal
        for (int q = 0; q < tp.world; ++q) st_release_sys(tp.flags[q] + tp.site * FLAG_WORDS_PER_SITE + tp.rank, next);
      }
      if (tm) tm[2] = globaltimer_ns();
    }
    // Rows this rank reduces: its own slice (two-shot: reduce-scatter, then the rows are
    // pushed to every rank) or all of them (one-shot: every rank reduces every row itself
    // and keeps the result local; cheaper for a handful of decode rows, one hop less).
    const int rows_per = (p.T + tp.world - 1) / tp.world;
    const int r0 = tp.one_shot ? 0 : tp.rank * rows_per;
    const int r1 = tp.one_shot ? p.T : min(p.T, r0 + rows_per);
    const int rows = max(r1 - r0, 0);
    const int nvec = H / 4;
    // G CTAs share one row when there are fewer rows than CTAs (each takes a column slice
    // and the slices exchange their sum of squares through tagged slots, in fixed order)
    // (only worth the exchange when there are far fewer rows than CTAs)
    int G = 1;
    if (rows > 0 && rows * 4 <= (int)gridDim.x) {
      G = min(min((int)gridDim.x / rows, 16), max(nvec / 64, 1));
    }
    G = max(G, (nvec + TP_KEEP * NUM_THREADS - 1) / (TP_KEEP * NUM_THREADS));  // a thread keeps at most TP_KEEP vectors of a row
    const int per = (nvec + G - 1) / G;
    const uint32_t tag = tp_epoch * 1024u + (uint32_t)tp.site + 1u;  // unique per (site, call) on this rank
    unsigned long long* ss_slots = reinterpret_cast<unsigned long long*>(tp.flags[tp.rank] + 768 * FLAG_WORDS_PER_SITE);
    // every rank pushed its partial rows into this rank's receive buffer [source rank][row][hidden]
    const float* recv = tp.part[tp.rank] + tp.part_offset;
    const size_t src_stride = (size_t)(tp.one_shot ? p.T : rows_per) * H;
    bool waited = false, ok = true;
    for (int unit = blockIdx.x; unit < rows * G; unit += gridDim.x) {
      if (!waited) {
        if (threadIdx.x == 0) *s_ok = wait_epochs(myflags, tp.world, next, tp.wait_ns, p.status, 3u) ? 1u : 0u;
        if (tm) tm[3] = globaltimer_ns();
        __syncthreads();
        ok = *s_ok != 0u;
        waited = true;
      }
      if (!ok) break;
      const int row = r0 + unit / G, g = unit % G;
      const int lo = g * per, hi = min(nvec, lo + per);
      const int iters = (hi - lo + NUM_THREADS - 1) / NUM_THREADS;
      bf16* res_row = tp.residual + (size_t)row * tp.ld_res;
      const float* src_row = recv + (size_t)(row - r0) * H;
      uint2 keep[TP_KEEP];  // this thread's updated residual values (4 bf16 each), reused by pass 2
      float ss;
      switch (tp.world) {
        case 1: ss = tp_sum_rows<1>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 2: ss = tp_sum_rows<2>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 3: ss = tp_sum_rows<3>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 4: ss = tp_sum_rows<4>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 5: ss = tp_sum_rows<5>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 6: ss = tp_sum_rows<6>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        case 7: ss = tp_sum_rows<7>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
        default: ss = tp_sum_rows<8>(src_row, src_stride, res_row, lo, hi, iters, keep); break;
      }
      ss = block_sum(ss, red);
      if (G > 1) {
        unsigned long long* slot = ss_slots + (size_t)(row - r0) * 16;
        if (threadIdx.x == 0) {
          const unsigned long long v = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(ss);
          asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(slot + g), "l"(v) : "memory");
        }
        float tot = 0.f;
        if (threadIdx.x == 0) {
          const uint64_t t0 = globaltimer_ns();
          for (int j = 0; j < G; ++j) {
            unsigned long long v;
            uint32_t spins = 0;
            while (true) {
              asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot + j) : "memory");
              if ((uint32_t)(v >> 32) == tag) break;
              if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > tp.wait_ns) {
                atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (10u << 8));
                break;
              }
            }
            tot += __uint_as_float((uint32_t)v);
          }
          red[33] = tot;
        }
        __syncthreads();
        ss = red[33];
      }
      const float inv = rsqrtf(ss / (float)H + tp.eps);
      // pass 2: normalise the values kept in registers and deliver them
#pragma unroll
      for (int it = 0; it < TP_KEEP; ++it) {
        const int i = lo + threadIdx.x + it * NUM_THREADS;
        if (it < iters && i < hi) {
          const uint2 kv = keep[it];
          const float2 f0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&kv.x)), f1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&kv.y));
          const uint2 wv = *(reinterpret_cast<const uint2*>(tp.norm_w) + i);
          float2 w0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&wv.x)), w1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&wv.y));
          if (tp.offset) {
            w0.x += 1.f;
            w0.y += 1.f;
            w1.x += 1.f;
            w1.y += 1.f;
          }
          uint2 packed;
          bf162 o0 = __floats2bfloat162_rn(f0.x * inv * w0.x, f0.y * inv * w0.y);
          bf162 o1 = __floats2bfloat162_rn(f1.x * inv * w1.x, f1.y * inv * w1.y);
          packed.x = *reinterpret_cast<uint32_t*>(&o0);
          packed.y = *reinterpret_cast<uint32_t*>(&o1);
          if (tp.one_shot) {
            reinterpret_cast<uint2*>(tp.xout[tp.rank] + (size_t)row * H)[i] = packed;
          } else {
#pragma unroll
            for (int q = 0; q < MAX_RANKS; ++q)
              if (q < tp.world) reinterpret_cast<uint2*>(tp.xout[q] + (size_t)row * H)[i] = packed;
          }
        }
      }
    }
    // phase 2 done: the last CTA publishes "rows of this rank delivered" and advances the epoch
    __syncthreads();
    if (tm) tm[4] = globaltimer_ns();
    if (threadIdx.x == 0) {
      if (!tp.one_shot) __threadfence_system();
      const uint32_t old = atomicAdd(&myflags[18], 1u);
      if (old == gridDim.x - 1) {
        myflags[18] = 0u;
        if (!tp.one_shot)
          for (int q = 0; q < tp.world; ++q) st_release_sys(tp.flags[q] + tp.site * FLAG_WORDS_PER_SITE + 8 + tp.rank, next);
        __threadfence();
        *((volatile uint32_t*)&myflags[16]) = next;
      }
      if (tm) tm[5] = globaltimer_ns();
    }
  }
}

// Stand-alone wait for consumers of all-gathered rows that are not this GEMM.
__global__ void tp_wait_kernel(WaitSpec w, uint32_t* status) {
  if (threadIdx.x == 0) {
    const uint32_t target = *((volatile const uint32_t*)(w.flags + 16));
    wait_epochs(w.flags + 8, w.world, target, w.wait_ns, status, 4u);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct DeviceInfo {
  int sms = 0;
  int max_smem = 0;
  bool attr_set = false;
  int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};  // co-resident clusters of size S at one CTA per SM (0 = not usable)
};
DeviceInfo g_dev[64];
std::mutex g_mu;

}  // namespace

// Row-major [rows, cols] bf16 matrix with row stride ld elements; box = [box_rows x 64].
int pg_make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols) {
  EncodeTiledFn enc = get_encode();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0, "TMA base address must be 16-byte aligned");
  PG_REQUIRE((ld * 2) % 16 == 0, "TMA row stride must be a multiple of 16 bytes (ld=%lld)", ld);
  PG_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_cols * 2 == 128, "unsupported TMA box %dx%d", box_rows, box_cols);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}

static int pick_bn(int T, int M, int sms) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  // large T: time ~ waves x (MMA time ~ bn, plus the fixed 128-row weight tile per stage)
  const int m_tiles = ceil_div(M, BM);
  int best = 256;
  long long best_cost = -1;
  for (int bn = 256; bn >= 128; bn -= 16) {
    const long long tiles = (long long)m_tiles * ceil_div(T, bn);
    const long long waves = (tiles + sms - 1) / sms;
    const long long cost = waves * (bn + 64);
    if (best_cost < 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

// Pick the k-split count that minimises (wave quantisation) x (partial-sum overhead).
static int pick_splits(int tiles, int kblocks, int bn, int sms) {
  if (tiles >= 4 * sms) return 1;
  if (bn > 64 && tiles * 2 > sms) return 1;  // wide tiles: the f32 partial round trip costs more than the idle SMs
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && kblocks / s < 4) break;
    long long items = (long long)tiles * s;
    long long waves = (items + sms - 1) / sms;
    double eff = (double)items / (double)(waves * sms);
    // a split adds 2 * bn * 128 * 4 bytes of L2 traffic per item on top of kblocks/s * 16 KB of weights
    double overhead = s > 1 ? (2.0 * bn * 128 * 4) / ((double)kblocks / s * A_BYTES) : 0.0;
    double cost = (1.0 + 0.5 * overhead) / eff;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// One-shot hint consumed by the next GEMM launched from this thread.
unsigned long long* g_gemm_timing = nullptr;  // profiling hook, see pg_gemm_set_timing
thread_local const void* t_pf_ptr = nullptr;
thread_local long long t_pf_bytes = 0;

// Cluster size for the distributed-shared-memory split-K (token tiles up to 64 wide):
// time ~ rounds x (k-blocks per CTA + a fixed per-item cost worth ~6 k-blocks of streaming).
static int pick_cluster(int tiles, int kblocks, const int* max_clusters) {
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 8; ++s) {
    if (max_clusters[s] <= 0) continue;
    if (s > 1 && kblocks / s < 4) break;
    const int rounds = ceil_div(tiles, max_clusters[s]);
    const double cost = (double)rounds * ((double)ceil_div(kblocks, s) + (s > 1 ? 6.0 : 4.0));
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

extern "C" int pg_gemm_workspace_bytes(int T, int M, int K, int device, long long* ws_bytes, long long* counter_bytes) {
  int sms = 0;
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  int bn = pick_bn(T, M, sms);
  int tiles = ceil_div(M, BM) * ceil_div(T, bn);
  int splits = pick_splits(tiles, ceil_div(K, BK), bn, sms);
  *ws_bytes = splits > 1 ? (long long)tiles * splits * bn * BM * 4 : 0;
  *counter_bytes = (long long)tiles * 4;
  return PG_OK;
}

// y[T, M] (row stride ldy) = x[T, K] (row stride ldx) * w[M, K]^T (row stride ldw).
// `ws`/`counters` are caller-provided scratch (see pg_gemm_workspace_bytes); the counters
// must be zero before the first use and are left zero by every completed launch.
// `force_splits` > 0 pins the k-split count (batch-invariant serving); 0 = heuristic.
static int gemm_impl(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                     void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status, int force_splits,
                     const TpFuse* tp, const WaitSpec* wait, cudaStream_t stream, int* plan_out = nullptr, const FuseSpec* fuse = nullptr) {
  PG_REQUIRE(T > 0 && M > 0 && K > 0, "gemm: empty problem %dx%dx%d", T, M, K);
  PG_REQUIRE(K % 8 == 0, "gemm: K=%d must be a multiple of 8 (16-byte TMA rows)", K);
  PG_REQUIRE(status != nullptr, "gemm: a device status word is required");
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  DeviceInfo& di = g_dev[dev & 63];
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!di.attr_set) {
      PG_CUDA(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
      PG_CUDA(cudaDeviceGetAttribute(&di.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_PLAIN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_PLAIN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_SWIGLU, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_SWIGLU, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_RESID_NORMW, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<EPI_RESID_NORMW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      di.max_clusters[1] = di.sms;
      const char* env = getenv("PEGAINFER_GEMM_CLUSTER");
      const bool use_clusters = !(env && env[0] == '0');
      for (int s = 2; s <= 8 && use_clusters; ++s) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)(s * di.sms));
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = (size_t)di.max_smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = (unsigned)s;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_tn_kernel<EPI_PLAIN, false>, &cfg) == cudaSuccess) di.max_clusters[s] = n;
        else (void)cudaGetLastError();
      }
      di.attr_set = true;
    }
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if (tp) p.tp = *tp;
  if (wait) p.wait = *wait;
  if (fuse) p.fuse = *fuse;
  p.bn = pick_bn(T, M, di.sms);
  p.m_tiles = ceil_div(M, BM);
  p.n_tiles = ceil_div(T, p.bn);
  p.kblocks = ceil_div(K, BK);
  const int tiles = p.m_tiles * p.n_tiles;
  p.cluster = 1;
  p.splits = 0;
  if (p.bn <= 64 && force_splits <= 8 && di.max_clusters[2] > 0) {
    // narrow token tiles: the k-splits of a tile form one cluster and reduce on chip
    const int s = force_splits > 0 ? (di.max_clusters[force_splits] > 0 ? force_splits : 0) : pick_cluster(tiles, p.kblocks, di.max_clusters);
    if (s > 0 && s <= p.kblocks) {
      p.splits = s;
      p.cluster = s;
    }
  }
  if (p.splits == 0) {
    p.splits = force_splits > 0 ? force_splits : pick_splits(tiles, p.kblocks, p.bn, di.sms);
    if (p.splits > p.kblocks) p.splits = p.kblocks;
    if (force_splits <= 0) {
      // never outgrow the caller's scratch: fewer splits only cost load balance
      while (p.splits > 1 && (ws == nullptr || ws_bytes < (long long)tiles * p.splits * p.bn * BM * 4 || counter_bytes < (long long)tiles * 4)) --p.splits;
    }
    if (p.splits > 1) {
      PG_REQUIRE(ws != nullptr && ws_bytes >= (long long)tiles * p.splits * p.bn * BM * 4, "gemm: workspace too small for %d splits", p.splits);
      PG_REQUIRE(counters != nullptr && counter_bytes >= (long long)tiles * 4, "gemm: counter buffer too small");
    }
  }
  if (fuse && fuse->epi != EPI_PLAIN && p.cluster <= 1) {
    pg_set_error("gemm: the fused epilogue needs the on-chip split-K path (T <= 64 and a cluster plan); T=%d M=%d K=%d plans cluster=%d", T, M, K, p.cluster);
    return PG_ERR_UNSUPPORTED;
  }
  const int stage_bytes = A_BYTES + p.bn * 128;
  const int tail = (2 * MAX_STAGES + 6) * 8 + 64 + 1024;  // barriers, flags, 256 floats of per-token scales
  const int red_bytes = p.cluster > 1 ? (p.bn + 8) * BM * 4 : 0;  // S slots of ceil(bn / S) columns
  p.stages = (di.max_smem - 1024 - tail - red_bytes) / stage_bytes;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  PG_REQUIRE(p.stages >= 2, "gemm: not enough shared memory for a 2-stage pipeline");
  uint32_t cols = 32;
  while (cols < (uint32_t)(2 * p.bn)) cols <<= 1;
  p.tmem_cols = cols;
  p.y = y_is_f32 ? nullptr : (bf16*)y;
  p.y_f32 = y_is_f32 ? (float*)y : nullptr;
  p.ldy = ldy;
  p.M = M;
  p.T = T;
  p.K = K;
  p.ws = (float*)ws;
  p.counters = (uint32_t*)counters;
  p.status = (uint32_t*)status;
  p.timing = g_gemm_timing;
  {
    static int rot = -1;
    if (rot < 0) {
      const char* e = getenv("PEGAINFER_GEMM_ROTATE");
      rot = (e && e[0] == '0') ? 0 : 1;
    }
    p.rotate = rot;
  }
  if (plan_out == nullptr) {
    p.pf_ptr = (const uint8_t*)t_pf_ptr;
    p.pf_bytes = (t_pf_ptr && T <= 256) ? t_pf_bytes : 0;  // only the weight-streaming regime has idle HBM time to fill
    t_pf_ptr = nullptr;
    t_pf_bytes = 0;
  }
  if (plan_out != nullptr) {
    const int total_items = tiles * p.splits;
    plan_out[0] = p.bn;
    plan_out[1] = p.splits;
    plan_out[2] = p.cluster;
    plan_out[3] = p.cluster > 1 ? (tiles < di.max_clusters[p.cluster] ? tiles : di.max_clusters[p.cluster]) * p.cluster : (total_items < di.sms ? total_items : di.sms);
    plan_out[4] = p.stages;
    plan_out[5] = di.max_clusters[p.cluster];
    return PG_OK;
  }
  CUtensorMap tm_w, tm_x;
  int rc = pg_make_tmap_bf16_2d(&tm_w, w, M, K, ldw, BM, BK);
  if (rc) return rc;
  rc = pg_make_tmap_bf16_2d(&tm_x, x, T, K, ldx, p.bn, BK);
  if (rc) return rc;
  const int total = tiles * p.splits;
  int grid = total < di.sms ? total : di.sms;
  if (p.cluster > 1) grid = (tiles < di.max_clusters[p.cluster] ? tiles : di.max_clusters[p.cluster]) * p.cluster;
  const size_t smem = 1024 + (size_t)p.stages * stage_bytes + red_bytes + tail;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (p.cluster > 1) {
    at[na].id = cudaLaunchAttributeClusterDimension;
    at[na].val.clusterDim.x = (unsigned)p.cluster;
    at[na].val.clusterDim.y = 1;
    at[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = (unsigned)na;
  if (pdl_enabled()) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.numAttrs = (unsigned)na;
  const bool inv = p.fuse.in_ssp != nullptr;
  cudaError_t le;
  switch (p.fuse.epi * 2 + (inv ? 1 : 0)) {
    case 1: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_PLAIN, true>, tm_w, tm_x, p); break;
    case 2: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_SWIGLU, false>, tm_w, tm_x, p); break;
    case 3: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_SWIGLU, true>, tm_w, tm_x, p); break;
    case 4: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_RESID_NORMW, false>, tm_w, tm_x, p); break;
    case 5: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_RESID_NORMW, true>, tm_w, tm_x, p); break;
    default: le = cudaLaunchKernelEx(&cfg, gemm_bf16_tn_kernel<EPI_PLAIN, false>, tm_w, tm_x, p); break;
  }
  PG_CUDA(le);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// How a problem would be launched on the current device (for tests, reports and tuning):
// out = {bn, splits, cluster, grid, stages, max co-resident clusters of that size}.
// The next GEMM launched from the calling thread also pulls `bytes` at `ptr` (16-byte
// aligned; normally the leading part of the weight matrix of the GEMM that follows it in
// the stream) into L2.  bytes <= 0 or ptr == nullptr clears the hint.
extern "C" void pg_gemm_prefetch_next(const void* ptr, long long bytes) {
  if (ptr == nullptr || bytes <= 0 || ((uintptr_t)ptr & 15) != 0) {
    t_pf_ptr = nullptr;
    t_pf_bytes = 0;
    return;
  }
  t_pf_ptr = ptr;
  t_pf_bytes = bytes;
}

// Profiling hook: a device buffer of 16 x uint64 per CTA (148 CTAs at most) that every
// following GEMM launch fills with globaltimer stamps of its phases: [0] entry, [1] prologue
// done, [2] predecessor complete, [3] all loads issued, [4] first stage landed, [5] last MMA
// committed, [6] accumulator ready, [7] partial stored, [8] all partials of the cluster
// stored, [9] reduced and written, [10] roles done, [11] cluster released.  nullptr = off.
extern "C" void pg_gemm_set_timing(void* buf) { g_gemm_timing = (unsigned long long*)buf; }

extern "C" int pg_gemm_plan(int T, int M, int K, int force_splits, int* out) {
  PG_REQUIRE(out != nullptr, "gemm plan: null output");
  void* fake = reinterpret_cast<void*>(uintptr_t(256));
  return gemm_impl(fake, fake, fake, 0, T, M, K, K, K, M, fake, 1ll << 40, fake, 1ll << 40, fake, force_splits, nullptr, nullptr, nullptr, out);
}

static unsigned long long* g_tp_timing = nullptr;
static int g_tp_last_site = 0;
// Profiling hook: device buffer of 8 x uint64 per site (nullptr switches it off).
extern "C" void pg_tp_set_timing(void* buf) { g_tp_timing = (unsigned long long*)buf; }

extern "C" int pg_gemm_bf16_tn(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx, long long ldw,
                               long long ldy, void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status,
                               int force_splits, cudaStream_t stream) {
  // tensor-bound problems go to the two-SM kernel; a pinned split count (batch-invariant
  // serving) keeps every problem size on this one kernel
  if (!y_is_f32 && force_splits <= 0 && pg_gemm2sm_eligible(T, M, K)) return pg_gemm2sm_bf16_tn(x, w, y, T, M, K, ldx, ldw, ldy, status, stream);
  return gemm_impl(x, w, y, y_is_f32, T, M, K, ldx, ldw, ldy, ws, ws_bytes, counters, counter_bytes, status, force_splits, nullptr, nullptr, stream);
}

// Same GEMM, but X rows are being all-gathered into `x` by peers: the TMA producer streams
// weight tiles first, then waits for every rank's rows-delivered epoch in `wait_flags` (the
// local flag block of the producing site).
extern "C" int pg_gemm_bf16_tn_after_gather(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx,
                                            long long ldw, long long ldy, void* ws, long long ws_bytes, void* counters, long long counter_bytes,
                                            void* status, const void* wait_flags, int world, unsigned long long wait_ns, cudaStream_t stream) {
  WaitSpec ws_;
  ws_.flags = (const uint32_t*)wait_flags;
  ws_.world = world;
  ws_.wait_ns = wait_ns;
  ws_.timing = g_tp_timing ? g_tp_timing + g_tp_last_site * 8 : nullptr;
  return gemm_impl(x, w, y, y_is_f32, T, M, K, ldx, ldw, ldy, ws, ws_bytes, counters, counter_bytes, status, 0, nullptr,
                   wait_flags ? &ws_ : nullptr, stream);
}

// Row-parallel projection fused with its collective:  partial = a[T, K_local] * w[hidden, K_local]^T
// (tcgen05 tiles, f32) -> reduce-scatter over peer memory (fixed rank order) -> + residual ->
// RMSNorm -> all-gather of the normalised rows into every rank's `xout`.  `part`, `xout`,
// `flags` are arrays of `world` peer-mapped pointers (index = rank).  Consumers of `xout`
// wait on flags[rank] + site * 32 (pg_gemm_bf16_tn_after_gather or pg_tp_wait).
extern "C" int pg_tp_gemm_rs_norm_ag(const void* a, const void* w, int T, int hidden, int K, long long lda, long long ldw, void* const* part,
                                     void* const* xout, void* const* flags, int rank, int world, int site, void* residual, long long ld_res,
                                     const void* norm_w, float eps, int offset, int one_shot, long long part_offset, unsigned long long wait_ns,
                                     void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status, cudaStream_t stream) {
  PG_REQUIRE(world >= 1 && world <= MAX_RANKS && rank >= 0 && rank < world, "tp gemm: bad rank %d / world %d", rank, world);
  PG_REQUIRE(hidden % 8 == 0 && hidden <= 16 * TP_KEEP * NUM_THREADS * 4, "tp gemm: hidden %d must be a multiple of 8 and <= %d", hidden, 16 * TP_KEEP * NUM_THREADS * 4);
  PG_REQUIRE(((uintptr_t)residual & 7) == 0 && ld_res % 4 == 0 && ((uintptr_t)norm_w & 7) == 0, "tp gemm: residual rows and norm weights must be 8-byte aligned");
  PG_REQUIRE(site >= 0 && site < 768, "tp gemm: site %d out of range", site);
  TpFuse tp;
  memset(&tp, 0, sizeof(tp));
  tp.enabled = 1;
  tp.rank = rank;
  tp.world = world;
  tp.site = site;
  for (int q = 0; q < world; ++q) {
    tp.part[q] = (float*)part[q];
    tp.xout[q] = (bf16*)xout[q];
    tp.flags[q] = (uint32_t*)flags[q];
  }
  tp.residual = (bf16*)residual;
  tp.ld_res = ld_res;
  tp.norm_w = (const bf16*)norm_w;
  tp.eps = eps;
  tp.offset = offset;
  tp.one_shot = one_shot;
  tp.part_offset = part_offset;
  tp.wait_ns = wait_ns;
  tp.timing = g_tp_timing;
  g_tp_last_site = site;
  return gemm_impl(a, w, (float*)part[rank] + part_offset, 1, T, hidden, K, lda, ldw, hidden, ws, ws_bytes, counters, counter_bytes, status, 0, &tp, nullptr, stream);
}

// The decode-chain form of the GEMM (T <= 64): optional deferred-RMSNorm scaling of the input rows
// (`in_ssp` [in_parts][T] sums of squares written by the producer, nullptr = none) and a fused
// epilogue: 0 plain, 1 SwiGLU over interleaved (gate, up) weight rows (y is [T, M / 2]), 2 residual
// add + norm-weight product (y = xw [T, M], `residual` updated in place, `out_ssp` [ceil(M / 128)][T]
// written).  Returns PG_ERR_UNSUPPORTED when the problem does not plan onto the on-chip split-K path;
// the caller then runs the separate kernels.
extern "C" int pg_gemm_bf16_tn_fused(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                                     const void* in_ssp, int in_parts, int in_ld, int in_width, float in_eps, int epi, void* residual, long long ld_res,
                                     const void* norm_w, int norm_offset, void* out_ssp, int out_ld, void* ws, long long ws_bytes, void* counters,
                                     long long counter_bytes, void* status, cudaStream_t stream) {
  PG_REQUIRE(epi >= EPI_PLAIN && epi <= EPI_RESID_NORMW, "gemm fused: unknown epilogue %d", epi);
  PG_REQUIRE(T <= 64, "gemm fused: built for decode steps of at most 64 token rows, got %d", T);
  PG_REQUIRE(in_ssp == nullptr || (in_parts > 0 && in_width > 0 && in_ld >= in_parts && in_ld % 4 == 0 && ((uintptr_t)in_ssp & 15) == 0),
             "gemm fused: input scale needs its part count, width and a 16-byte aligned row pitch that is a multiple of 4");
  if (epi == EPI_SWIGLU) PG_REQUIRE(M % 4 == 0 && ldy % 2 == 0, "gemm fused: SwiGLU needs M %% 4 == 0");
  if (epi == EPI_RESID_NORMW) {
    PG_REQUIRE(M % BM == 0, "gemm fused: residual + norm epilogue needs M (%d) to be a multiple of %d", M, BM);
    PG_REQUIRE(out_ld >= M / BM, "gemm fused: out_ssp rows hold %d entries, %d weight tiles", out_ld, M / BM);
    PG_REQUIRE(residual && norm_w && out_ssp && ld_res % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)residual & 7) == 0 && ((uintptr_t)norm_w & 7) == 0 && ((uintptr_t)y & 7) == 0,
               "gemm fused: residual, norm weight and output must be given and 8-byte aligned");
  }
  FuseSpec f;
  memset(&f, 0, sizeof(f));
  f.epi = epi;
  f.in_ssp = (const float*)in_ssp;
  f.in_parts = in_parts;
  f.in_ld = in_ld;
  f.in_width = in_width;
  f.in_eps = in_eps;
  f.residual = (bf16*)residual;
  f.ld_res = ld_res;
  f.norm_w = (const bf16*)norm_w;
  f.norm_offset = norm_offset;
  f.out_ssp = (float*)out_ssp;
  f.out_ld = out_ld;
  return gemm_impl(x, w, y, 0, T, M, K, ldx, ldw, ldy, ws, ws_bytes, counters, counter_bytes, status, 0, nullptr, nullptr, stream, nullptr, &f);
}

extern "C" int pg_tp_wait(const void* wait_flags, int world, unsigned long long wait_ns, void* status, cudaStream_t stream) {
  WaitSpec w_;
  w_.flags = (const uint32_t*)wait_flags;
  w_.world = world;
  w_.wait_ns = wait_ns;
  w_.timing = nullptr;
  tp_wait_kernel<<<1, 32, 0, stream>>>(w_, (uint32_t*)status);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// ---- peer memory plumbing (one process per GPU; handles travel through torch.distributed) ----
extern "C" int pg_symm_alloc(long long bytes, void** out) {
  PG_CUDA(cudaMalloc(out, (size_t)bytes));
  PG_CUDA(cudaMemset(*out, 0, (size_t)bytes));
  return PG_OK;
}
extern "C" int pg_symm_free(void* p) {
  PG_CUDA(cudaFree(p));
  return PG_OK;
}
extern "C" int pg_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  PG_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, sizeof(h));
  return PG_OK;
}
extern "C" int pg_ipc_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  PG_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return PG_OK;
}
extern "C" int pg_ipc_close(void* p) {
  PG_CUDA(cudaIpcCloseMemHandle(p));
  return PG_OK;
}

// ---------------------------------------------------------------------------------
// Allocation-free variant (see gemm_noalloc.h): same kernel, scratch inside the image.
// ---------------------------------------------------------------------------------
#include "gemm_noalloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer
// that a kernel could be given.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PG_NOALLOC_SCRATCH_BYTES];

static void* g_noalloc_ptr[64];
static bool g_noalloc_ready[64];
static std::mutex g_noalloc_mu;

extern "C" int pg_gemm_bf16_tn_noalloc(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                                       void* status, cudaStream_t stream) {
  PG_REQUIRE(T > 0 && M > 0 && K > 0, "gemm_noalloc: empty problem %dx%dx%d", T, M, K);
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  PG_REQUIRE(dev >= 0 && dev < 64, "gemm_noalloc: device ordinal %d out of range", dev);
  void* scratch = nullptr;
  int sms = 0;
  {
    // once per device, with that device current: resolve the device address of the array
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ready[dev]) {
      void* ptr = nullptr;
      PG_CUDA(cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch));
      PG_REQUIRE(ptr != nullptr, "gemm_noalloc: scratch symbol resolved to a null address");
      g_noalloc_ptr[dev] = ptr;
      g_noalloc_ready[dev] = true;
    }
    scratch = g_noalloc_ptr[dev];
  }
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int bn = pick_bn(T, M, sms);
  const long long tiles = (long long)ceil_div(M, BM) * ceil_div(T, bn);
  PG_REQUIRE(tiles <= PG_NOALLOC_MAX_TILES,
             "gemm_noalloc: %lld output tiles (M=%d, T=%d) exceed the built-in scratch limit of %d tiles; use pg_gemm_bf16_tn with caller scratch",
             tiles, M, T, (int)PG_NOALLOC_MAX_TILES);
  unsigned char* base = static_cast<unsigned char*>(scratch);
  // the counters must start at zero; the partial sums are fully written before they are read
  PG_CUDA(cudaMemsetAsync(base, 0, (size_t)tiles * 4, stream));
  return pg_gemm_bf16_tn(x, w, y, 0, T, M, K, ldx, ldw, ldy, base + PG_NOALLOC_COUNTER_BYTES,
                         (long long)PG_NOALLOC_SCRATCH_BYTES - PG_NOALLOC_COUNTER_BYTES, base, PG_NOALLOC_COUNTER_BYTES, status, 0, stream);
}
