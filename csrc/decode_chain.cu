// Decode chain: up to four dependent bf16 GEMMs of one transformer layer in ONE persistent
// kernel, for steps of at most 64 token rows.
//
//   o_proj -> (+ residual, RMSNorm) -> gate_up (SwiGLU) -> down -> (+ residual, RMSNorm) -> next qkv
//
// Launched as separate kernels, each of these GEMMs pays a fixed price around its weight
// stream: the completion latency between dependent kernels, the prologue, the latency of the
// first activation tile and the split-K tail -- measured ~9 us per GEMM on B200 while the
// stream itself takes 5 - 35 us.  Here one grid of one CTA per SM walks all phases:
//
//   * work split: a phase with `tiles` 128-row weight tiles on G CTAs gives every CTA
//     floor(tiles / G) whole tiles; the remaining tiles are cut stream-K style: their k-blocks,
//     laid end to end, are dealt out in equal contiguous ranges, so every CTA streams the same
//     number of bytes.  A range that does not cover a whole tile leaves an f32 partial in a
//     global scratch slot (at most two per CTA);
//   * a grid barrier (atomic counter, bounded spin) ends the GEMM part of a phase; the fix-up
//     then runs on all CTAs: partials are summed in CTA order (deterministic) and the phase's
//     epilogue is applied -- plain store, SwiGLU over interleaved (gate, up) rows, or residual add +
//     norm-weight product.  RMSNorm is deferred: the phase that adds the residual stores
//     xw = h * norm_w and per-(token, weight tile) sums of squares of h; the phase that consumes xw
//     multiplies each output element of token n by rsqrt(sum_tiles ssp[n][tile] / H + eps), so no
//     step ever needs a whole row in one place.  A second barrier publishes the phase's output;
//   * the weight producer never waits for a barrier: weights are constants, so while a CTA sits
//     in the fix-up of phase p its producer already fills the ring with the first weight tiles
//     of phase p + 1, and HBM stays busy across phase boundaries.  Weight tiles and token tiles
//     have separate rings and barriers for that reason.
//
//   warp 0  weight producer (TMA, 10-stage ring)      warp 1  token-tile producer (TMA, 6 stages)
//   warp 2  TMEM allocation + tcgen05.mma issue        warps 3..10 epilogue / fix-up
//
// Every wait is bounded and reports through the status word.  No TMA multicast, no clusters.
//
// Takes the place of the reference's per-op decode sequence GEMM -> fused_add_rms_norm -> GEMM
// -> silu_mul -> GEMM -> fused_add_rms_norm -> GEMM (pegainfer-qwen3/src/batch_decode.rs:265-399).
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int BN = 64;  // token tile = whole step
constexpr int W_BYTES = BM * BK * 2;
constexpr int X_BYTES = BN * BK * 2;
constexpr int NW = 10;
constexpr int NX = 6;
constexpr int EW = 8;                       // epilogue / fix-up warps
constexpr int THREADS = 96 + 32 * EW;
constexpr int MAX_PHASES = 4;
constexpr int SLOT_FLOATS = BN * BM;  // one partial tile, [token][128 weight rows] f32

enum { CH_PLAIN = 0, CH_SWIGLU = 1, CH_RESID_NORM = 2, CH_QKV_ROPE = 3 };
constexpr int MAX_SEGS = 6;  // partial segments of one remainder tile (k-blocks per tile / k-blocks per CTA, rounded up, plus one)

struct Phase {
  int M, K, kblocks, tiles;
  int full_rounds;  // whole tiles per CTA
  int rem_tiles;    // tiles cut into k-ranges
  int per_cta;      // k-blocks of the remainder per CTA (ceil)
  int epi;
  bf16* out;        // PLAIN / SWIGLU: [T, M] or [T, M / 2]; RESID_NORM: normalised rows [T, M]
  long long ld_out;
  const bf16* norm_w;  // RESID_NORM
  int norm_offset;
  const float* in_ssp;  // the input rows still owe their RMSNorm scale: [T][in_ld] sums of squares, in_parts per row (nullptr = none)
  int in_parts, in_ld, in_width;
  float in_eps;
  float* out_ssp;       // RESID_NORM: [T][out_ld], entry [token][weight tile]
  int out_ld;
  // QKV_ROPE (head_dim == 128, one weight tile = one head): per-head RMSNorm, RoPE, paged KV append
  const bf16* q_w;
  const bf16* k_w;
  const bf16* cos;
  const bf16* sin;
  const int* positions;
  const int* slots;
  bf16* kv;  // [pages, 2, page_size, Hkv, 128]
  int hq, hkv, rot, page_size, max_pos, has_qk_norm;
  long long num_slots;
  float qk_eps;
};

// Tensor parallelism: the row-parallel phases (residual + norm epilogue) sum their result over the
// ranks (either inside the switch with multimem.ld_reduce, or by pulling every rank's copy with plain peer
// loads over NVLink and adding in rank order; the pull has the lower latency for these 0.5 MB exchanges).  Every rank first reduces its own stream-K partials to a bf16 [T, M] partial in a buffer that
// is mapped on all ranks and bound to an NVSwitch multicast object; after a flag exchange each rank
// reads the sum over ranks with multimem.ld_reduce (reduced inside the switch, f32 accumulation) and
// finishes the epilogue on its own replicated copy of the residual.  Two partial buffers alternate
// between consecutive exchanges; exchange numbers (epochs) live in device memory, so CUDA-graph
// replays need no reset.
constexpr int TP_MAX_RANKS = 8;
constexpr int TP_FLAG_STRIDE = 160;  // flag words per source rank (one per CTA; at least the SM count)
constexpr int TP_EPOCH_WORD = TP_MAX_RANKS * TP_FLAG_STRIDE;
struct ChainTp {
  int world, rank;
  bf16* y_local[2];            // this rank's partial buffers [T, M]
  const bf16* y_mc[2];         // the same buffers through the multicast mapping
  const bf16* y_peer[TP_MAX_RANKS][2];  // every rank's partial buffers (peer mapped)
  int use_multimem;            // 1: sum with multimem.ld_reduce in the switch; 0: pull every rank's copy with plain peer loads and add in rank order
  uint32_t* flags_local;       // [TP_MAX_RANKS][TP_FLAG_STRIDE] latest exchange number announced by CTA c of each rank
  uint32_t* flags_peer[TP_MAX_RANKS];  // every rank's flag block (peer mapped)
  uint32_t* epoch;             // local word: exchanges completed by previous launches
  unsigned long long wait_ns;
};

__device__ __forceinline__ uint2 ld_relaxed_sys_u32x2(const void* addr) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ uint2 multimem_ld_reduce_bf16x4(const bf16* mc_addr) {
  uint2 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.bf16x2 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(mc_addr) : "memory");
  return v;
}

struct ChainParams {
  Phase ph[MAX_PHASES];
  int nphase;
  int T;
  int G;
  bf16* residual;
  long long ld_res;
  float eps;
  float* ws;           // [G][2][SLOT_FLOATS]
  uint32_t* counters;  // [3 * MAX_PHASES + 1], zero before the first launch, left zero by every launch
  ChainTp tp;
  uint32_t* status;
  unsigned long long* timing;  // optional profiling: 16 globaltimer stamps per CTA (nullptr = off)
};

struct Item {
  int tile, kb0, kb1, slot;  // slot < 0: the range covers the whole tile and the epilogue runs directly
};

// The idx-th work item of CTA `c` in a phase (idx counts from 0); false when there is none.
__device__ __forceinline__ bool get_item(const Phase& p, int G, int c, int idx, Item& it) {
  if (idx < p.full_rounds) {
    it.tile = idx * G + c;
    it.kb0 = 0;
    it.kb1 = p.kblocks;
    it.slot = -1;
    return true;
  }
  const int r = idx - p.full_rounds;
  if (r > 1 || p.rem_tiles == 0) return false;
  // 32-bit arithmetic throughout (the host checks rem_tiles * kblocks < 2^31): 64-bit division is emulated
  const int total = p.rem_tiles * p.kblocks;
  const int a = c * p.per_cta;
  const int b = min(a + p.per_cta, total);
  if (a >= b) return false;
  const int t0 = a / p.kblocks;
  const int e0 = min(b, (t0 + 1) * p.kblocks);
  if (r == 0) {
    it.tile = p.full_rounds * G + t0;
    it.kb0 = a - t0 * p.kblocks;
    it.kb1 = e0 - t0 * p.kblocks;
    it.slot = 0;
    return true;
  }
  if (e0 >= b) return false;
  it.tile = p.full_rounds * G + t0 + 1;
  it.kb0 = 0;
  it.kb1 = b - e0;
  it.slot = 1;
  return true;
}

__device__ __forceinline__ bool bar128(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until every CTA of the grid has arrived on `ctr` (bounded).
__device__ __forceinline__ bool grid_wait(const uint32_t* ctr, uint32_t G, uint32_t* status, volatile int* abort_flag, uint32_t site) {
  if (ld_acquire_gpu(ctr) >= G) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_gpu(ctr) >= G) return true;
    if ((++spins & 31u) == 0u) {
      if (*abort_flag) return false;
      if (*((volatile uint32_t*)status) != PG_ST_OK) {  // another CTA already gave up: do not wait out a second limit
        *abort_flag = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > PG_WAIT_LIMIT_NS) {
        atomicCAS(status, PG_ST_OK, PG_ST_TIMEOUT | (site << 8));
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void grid_arrive(uint32_t* ctr) {
  __threadfence();
  atomicAdd(ctr, 1u);
}

// What the fix-up of one unit (remainder tile, token) reads: the partial sums of the tile for that
// token (4 weight rows per lane), the residual / norm weight of those rows, this lane's share of the
// token's sums of squares.
struct FixIn {
  float4 a;
  uint2 rv, wv;
  float part;
};

__device__ __forceinline__ void fix_load(const ChainParams& p, const Phase& P, int u, int rem0, int lane, FixIn& f) {
  const int rt = u / p.T, n = u - rt * p.T;
  const int k_lo = rt * P.kblocks, k_hi = k_lo + P.kblocks - 1;
  const int c_lo = k_lo / P.per_cta, c_hi = k_hi / P.per_cta;
  f.a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int q0 = c_lo; q0 <= c_hi; q0 += MAX_SEGS) {  // one round for the shapes of real models
    float4 seg[MAX_SEGS];
#pragma unroll
    for (int q = 0; q < MAX_SEGS; ++q) {
      const int cc = q0 + q;
      seg[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cc <= c_hi) {
        const int slot = cc * P.per_cta >= k_lo ? 0 : 1;  // the tile is the CTA's first one iff its range starts inside the tile
        seg[q] = __ldcg(reinterpret_cast<const float4*>(p.ws + ((size_t)cc * 2 + slot) * SLOT_FLOATS + (size_t)n * BM) + lane);
      }
    }
#pragma unroll
    for (int q = 0; q < MAX_SEGS; ++q) {
      f.a.x += seg[q].x;
      f.a.y += seg[q].y;
      f.a.z += seg[q].z;
      f.a.w += seg[q].w;
    }
  }
  const int mcol = (rem0 + rt) * BM + lane * 4;
  f.rv = make_uint2(0u, 0u);
  f.wv = make_uint2(0u, 0u);
  if (P.epi == CH_RESID_NORM && mcol + 3 < P.M) {
    f.rv = __ldcg(reinterpret_cast<const uint2*>(p.residual + (size_t)n * p.ld_res + mcol));  // written by other SMs in an earlier phase
    f.wv = *reinterpret_cast<const uint2*>(P.norm_w + mcol);
  }
  f.part = 0.f;
  if (P.in_ssp != nullptr)
    for (int q = lane; q < P.in_parts; q += 32) f.part += __ldcg(P.in_ssp + (size_t)n * P.in_ld + q);
}

__device__ __forceinline__ void fix_finish(const ChainParams& p, const Phase& P, int u, int rem0, int lane, const FixIn& f, bool scale_input = true) {
  const int rt = u / p.T, n = u - rt * p.T;
  const int mcol = (rem0 + rt) * BM + lane * 4;
  float4 a = f.a;
  if (P.in_ssp != nullptr && scale_input) {
    // the token's inverse RMS: the lanes split the per-tile sums, the shuffle tree adds them in a fixed order
    const float inv = rsqrtf(warp_sum(f.part) / (float)P.in_width + P.in_eps);
    a.x *= inv, a.y *= inv, a.z *= inv, a.w *= inv;
  }
  if (P.epi == CH_QKV_ROPE) {
    // tile = head (head_dim 128): per-head RMSNorm, rotary embedding, q to its buffer, k / v into the paged cache
    const int h = rem0 + rt;
    if (h >= P.hq + 2 * P.hkv) return;
    float v[4] = {bf16_round(a.x), bf16_round(a.y), bf16_round(a.z), bf16_round(a.w)};
    long long slot = 0;
    if (h >= P.hq) {
      slot = P.slots[n];
      if (slot < 0 || slot >= P.num_slots) {
        if (lane == 0) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (3u << 8));
        return;
      }
    }
    const long long page = slot / P.page_size, off = slot % P.page_size;
    bf16* dst;
    if (h >= P.hq + P.hkv) {
      dst = P.kv + (((page * 2 + 1) * P.page_size + off) * P.hkv + (h - P.hq - P.hkv)) * BM;
    } else {
      int pos = P.positions[n];
      if (pos < 0 || pos >= P.max_pos) {
        if (lane == 0) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (4u << 8));
        pos = pos < 0 ? 0 : P.max_pos - 1;
      }
      if (P.has_qk_norm) {
        const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        const float invn = rsqrtf(ss / (float)BM + P.qk_eps);
        const uint2 nw = *reinterpret_cast<const uint2*>((h < P.hq ? P.q_w : P.k_w) + lane * 4);
        float2 w0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&nw.x)), w1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&nw.y));
        if (P.norm_offset) w0.x += 1.f, w0.y += 1.f, w1.x += 1.f, w1.y += 1.f;
        v[0] = bf16_round(v[0] * invn * w0.x);
        v[1] = bf16_round(v[1] * invn * w0.y);
        v[2] = bf16_round(v[2] * invn * w1.x);
        v[3] = bf16_round(v[3] * invn * w1.y);
      }
      const int half = P.rot >> 1;  // 64 when the whole head rotates: element i pairs with i +- 64 = lane +- 16
      const bf16* cs = P.cos + (long long)pos * half;
      const bf16* sn = P.sin + (long long)pos * half;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = lane * 4 + j;
        const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
        float o = v[j];
        if (i < half) o = v[j] * __bfloat162float(cs[i]) - other * __bfloat162float(sn[i]);
        else if (i < P.rot) o = v[j] * __bfloat162float(cs[i - half]) + other * __bfloat162float(sn[i - half]);
        v[j] = o;
      }
      dst = h < P.hq ? P.out + ((size_t)n * P.hq + h) * BM : P.kv + (((page * 2 + 0) * P.page_size + off) * P.hkv + (h - P.hq)) * BM;
    }
    const bf162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst + lane * 4) = pk;
    return;
  }
  if (mcol + 3 >= P.M) return;
  if (P.epi == CH_SWIGLU) {
    const float g0 = bf16_round(a.x), u0 = bf16_round(a.y), g1 = bf16_round(a.z), u1 = bf16_round(a.w);
    const bf162 o = __floats2bfloat162_rn(bf16_round(g0 / (1.f + __expf(-g0))) * u0, bf16_round(g1 / (1.f + __expf(-g1))) * u1);
    *reinterpret_cast<bf162*>(P.out + (size_t)n * P.ld_out + (mcol >> 1)) = o;
  } else if (P.epi == CH_RESID_NORM) {
    const float2 r0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&f.rv.x)), r1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&f.rv.y));
    const bf162 h0 = __floats2bfloat162_rn(a.x + r0.x, a.y + r0.y), h1 = __floats2bfloat162_rn(a.z + r1.x, a.w + r1.y);
    uint2 hp;
    hp.x = *reinterpret_cast<const uint32_t*>(&h0);
    hp.y = *reinterpret_cast<const uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(p.residual + (size_t)n * p.ld_res + mcol) = hp;
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
    float2 w0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&f.wv.x)), w1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&f.wv.y));
    if (P.norm_offset) w0.x += 1.f, w0.y += 1.f, w1.x += 1.f, w1.y += 1.f;
    const bf162 x0 = __floats2bfloat162_rn(f0.x * w0.x, f0.y * w0.y), x1 = __floats2bfloat162_rn(f1.x * w1.x, f1.y * w1.y);
    uint2 xp;
    xp.x = *reinterpret_cast<const uint32_t*>(&x0);
    xp.y = *reinterpret_cast<const uint32_t*>(&x1);
    *reinterpret_cast<uint2*>(P.out + (size_t)n * P.ld_out + mcol) = xp;
    const float ss = warp_sum(f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y);  // M is a multiple of 128: no lane left early
    if (lane == 0) P.out_ssp[(size_t)n * P.out_ld + rem0 + rt] = ss;
  } else {
    const bf162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(P.out + (size_t)n * P.ld_out + mcol) = pk;
  }
}

struct TMaps {
  CUtensorMap w[MAX_PHASES];
  CUtensorMap x[MAX_PHASES];
};

__global__ void __launch_bounds__(THREADS, 1) decode_chain_kernel(const __grid_constant__ TMaps tm, const ChainParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* wring = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* xring = wring + NW * W_BYTES;
  uint64_t* wfull = reinterpret_cast<uint64_t*>(xring + NX * X_BYTES);
  uint64_t* wempty = wfull + NW;
  uint64_t* xfull = wempty + NW;
  uint64_t* xempty = xfull + NX;
  uint64_t* tfull = xempty + NX;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_inv = reinterpret_cast<float*>(tmem_slot + 4);  // [BN] inverse RMS of the input rows of the current phase (whole-tile epilogues)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x, G = p.G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NW; ++s) {
      mbar_init(&wfull[s], 1);
      mbar_init(&wempty[s], 1);
    }
    for (int s = 0; s < NX; ++s) {
      mbar_init(&xfull[s], 1);
      mbar_init(&xempty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EW);
    }
    *abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < p.nphase; ++i) {
      tma_prefetch_desc(&tm.w[i]);
      tma_prefetch_desc(&tm.x[i]);
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // ---- weight producer: never waits for another CTA ----
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_first();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        const Phase& P = p.ph[ph];
        Item it;
        for (int idx = 0; ok && get_item(P, G, c, idx, it); ++idx) {
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            if (!mbar_wait(&wempty[stage], phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&wfull[stage], (uint32_t)W_BYTES);
            tma_load_2d(wring + stage * W_BYTES, &tm.w[ph], &wfull[stage], kb * BK, it.tile * BM, pol);
            if (++stage == NW) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- token-tile producer: the input of phase ph exists after the fix-up of phase ph - 1 ----
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      pdl_wait();
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        const Phase& P = p.ph[ph];
        if (ph > 0) {
          ok = grid_wait(p.counters + 3 * (ph - 1) + 2, (uint32_t)G, p.status, abort_flag, 20u + (uint32_t)ph);
          fence_proxy_async_all();  // rows written by other SMs' ordinary stores, read by the bulk-copy engine
        }
        Item it;
        for (int idx = 0; ok && get_item(P, G, c, idx, it); ++idx) {
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            if (!mbar_wait(&xempty[stage], phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&xfull[stage], (uint32_t)X_BYTES);
            tma_load_2d(xring + stage * X_BYTES, &tm.x[ph], &xfull[stage], kb * BK, 0, pol);
            if (++stage == NX) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 2) {
    // ---- MMA issue ----
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
      int ws = 0, xs = 0, acc = 0;
      uint32_t wph = 0, xph = 0, acc_phase = 0;
      bool ok = true;
      for (int ph = 0; ph < p.nphase && ok; ++ph) {
        const Phase& P = p.ph[ph];
        Item it;
        for (int idx = 0; ok && get_item(P, G, c, idx, it); ++idx) {
          if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          for (int kb = it.kb0; kb < it.kb1; ++kb) {
            if (!mbar_wait(&wfull[ws], wph, abort_flag) || !mbar_wait(&xfull[xs], xph, abort_flag)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(wring + ws * W_BYTES);
            const uint32_t b_addr = smem_u32(xring + xs * X_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_ss(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (kb > it.kb0 || k > 0) ? 1u : 0u);
            umma_commit(&wempty[ws]);
            umma_commit(&xempty[xs]);
            if (++ws == NW) {
              ws = 0;
              wph ^= 1u;
            }
            if (++xs == NX) {
              xs = 0;
              xph ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit(&tfull[acc]);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ---- epilogue and fix-up: warps 3..10; warp w may touch TMEM lanes 32 * (w % 4) .. + 31 ----
    const int wq = warp & 3;
    const int r = wq * 32 + lane;   // weight row inside the tile = TMEM lane
    const int et = threadIdx.x - 96;  // 0 .. 32 * EW - 1
    const int ew = et >> 5;           // 0 .. EW - 1; warps ew and ew + 4 share a TMEM lane quarter and split the token columns
    const int col0 = (ew >> 2) * (BN / 2), col1 = col0 + BN / 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    unsigned long long* ts = (p.timing && et == 0) ? p.timing + (size_t)c * 16 : nullptr;
    if (ts) ts[0] = globaltimer_ns();
    pdl_wait();
    // tensor parallel: exchanges completed before this launch (written by the previous launch's last CTA)
    const uint32_t tp_epoch = p.tp.world > 1 ? *((volatile uint32_t*)p.tp.epoch) : 0u;
    int tp_sites = 0;
    if (ts) ts[1] = globaltimer_ns();
    for (int ph = 0; ph < p.nphase; ++ph) {
      const Phase& P = p.ph[ph];
      Item it;
      if (P.in_ssp != nullptr && P.full_rounds > 0 && ok) {
        // whole-tile epilogues need every token's inverse RMS: the sums of squares come from the previous
        // phase's fix-up on other CTAs, complete once its second barrier is full
        bool w_ok = true;
        if (et == 0 && ph > 0) w_ok = grid_wait(p.counters + 3 * (ph - 1) + 2, (uint32_t)G, p.status, abort_flag, 30u + (uint32_t)ph);
        ok = bar128(w_ok);
        if (ok && et < 2 * BN) {
          const int n = et >> 1, half = et & 1;  // two threads per token
          const int per = (P.in_parts + 1) >> 1;
          const int q0 = half * per, q1 = min(P.in_parts, q0 + per);
          float ss = 0.f;
          if (n < p.T)
            for (int q = q0; q < q1; ++q) ss += __ldcg(P.in_ssp + (size_t)n * P.in_ld + q);
          const float other = __shfl_xor_sync(0xffffffffu, ss, 1);
          const float tot = half ? other + ss : ss + other;
          if (half == 0) s_inv[n] = rsqrtf(tot / (float)P.in_width + P.in_eps);
        }
        bar128(true);
      }
      const bool scale = P.in_ssp != nullptr;
      for (int idx = 0; ok && get_item(P, G, c, idx, it); ++idx) {
        ok = bar128(mbar_wait(&tfull[acc], acc_phase, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * BN);
        const int m = it.tile * BM + r;
        if (it.slot >= 0) {
          // partial: [token][128 rows] f32, coalesced across the warp
          float* dst = p.ws + ((size_t)c * 2 + it.slot) * SLOT_FLOATS + r;
#pragma unroll
          for (int cc = col0; cc < col1; cc += 16) {
            uint32_t v[16];
            tmem_ld16(t_row + cc, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (cc + j < p.T) dst[(size_t)(cc + j) * BM] = __uint_as_float(v[j]);
          }
        } else if (P.epi == CH_SWIGLU) {
          // whole tile: lanes (2i, 2i + 1) hold (gate_i, up_i); the even lane finishes the even columns
          // of a pair of columns, the odd lane the odd ones
#pragma unroll
          for (int cc = col0; cc < col1; cc += 16) {
            uint32_t v[16];
            tmem_ld16(t_row + cc, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              // exchange: even lane sends its gate of column j+1 and receives the up of column j
              const float mine0 = __uint_as_float(v[j]), mine1 = __uint_as_float(v[j + 1]);
              const float send = (lane & 1) ? mine0 : mine1;
              const float got = __shfl_xor_sync(0xffffffffu, send, 1);
              const float g = (lane & 1) ? got : mine0;
              const float u = (lane & 1) ? mine1 : got;
              const int n = cc + j + (lane & 1);
              if (n < p.T && m < P.M) {
                const float sc = scale ? s_inv[n] : 1.f;
                const float gb = bf16_round(g * sc), ub = bf16_round(u * sc);
                P.out[(size_t)n * P.ld_out + (m >> 1)] = __float2bfloat16(bf16_round(gb / (1.f + __expf(-gb))) * ub);
              }
            }
          }
        } else {
          // whole tile, plain store
#pragma unroll
          for (int cc = col0; cc < col1; cc += 16) {
            uint32_t v[16];
            tmem_ld16(t_row + cc, v);
            tmem_ld_wait();
            if (m < P.M) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (cc + j < p.T) P.out[(size_t)(cc + j) * P.ld_out + m] = __float2bfloat16(__uint_as_float(v[j]) * (scale ? s_inv[cc + j] : 1.f));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      // ---- all tiles / partials of this CTA are stored: first grid barrier of the phase ----
      uint32_t* bar_a = p.counters + 3 * ph;  // [3ph] partials stored, [3ph + 1] spare, [3ph + 2] output complete
      uint32_t* bar_b = bar_a + 2;
      ok = bar128(ok);
      if (ts) ts[2 + 3 * ph] = globaltimer_ns();  // this CTA's tiles and partials are stored
      if (et == 0) grid_arrive(bar_a);
      const int rem0 = P.full_rounds * G;  // first remainder tile
      const bool need_fix = P.rem_tiles > 0;
      if (need_fix) {
        bool w_ok = true;
        if (et == 0) w_ok = grid_wait(bar_a, (uint32_t)G, p.status, abort_flag, 10u + (uint32_t)ph);
        ok = bar128(ok && w_ok);
      }
      if (ts) ts[3 + 3 * ph] = globaltimer_ns();  // every CTA's partials are visible
      const bool tp_reduce = p.tp.world > 1 && P.epi == CH_RESID_NORM;
      if (ok && need_fix && tp_reduce) {
        // ---- tensor parallel row phase: local partials -> this rank's bf16 partial -> sum over ranks in the switch ----
        const int par = (int)((tp_epoch + (uint32_t)tp_sites) & 1u);
        const uint32_t e = tp_epoch + (uint32_t)tp_sites + 1u;
        bf16* y_loc = p.tp.y_local[par];
        const int units = P.rem_tiles * p.T;
        for (int u = c * EW + ew; u < units; u += 2 * EW * G) {
          const int u2 = u + EW * G;
          const bool two = u2 < units;
          FixIn f1, f2;
          fix_load(p, P, u, rem0, lane, f1);
          if (two) fix_load(p, P, u2, rem0, lane, f2);
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (k == 1 && !two) break;
            const int uu = k ? u2 : u;
            const FixIn& f = k ? f2 : f1;
            const int rt = uu / p.T, n = uu - rt * p.T;
            const int mcol = (rem0 + rt) * BM + lane * 4;
            float4 a = f.a;
            if (P.in_ssp != nullptr) {
              const float inv = rsqrtf(warp_sum(f.part) / (float)P.in_width + P.in_eps);
              a.x *= inv, a.y *= inv, a.z *= inv, a.w *= inv;
            }
            const bf162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            if (mcol + 3 < P.M) *reinterpret_cast<uint2*>(y_loc + (size_t)n * P.M + mcol) = pk;
          }
        }
        // This CTA's units of the rank partial are stored.  The same CTA index owns the same units on
        // every rank (same shapes, same grid), so the exchange is CTA to CTA: announce to CTA c of every
        // rank, wait for CTA c of every rank, no grid-wide step in between.
        ok = bar128(ok);
        if (et == 0) {
          bool w_ok = ok;
          if (ts) ts[13] = globaltimer_ns();  // rank partial of this CTA stored
          __threadfence_system();              // one fence for all flag stores below (a release store each would pay it per peer)
          for (int q = 0; q < p.tp.world; ++q)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.tp.flags_peer[q] + p.tp.rank * TP_FLAG_STRIDE + c), "r"(e) : "memory");
          if (ts) ts[14] = globaltimer_ns();  // announced
          const uint64_t t0 = globaltimer_ns();
          for (int q = 0; q < p.tp.world && w_ok; ++q) {
            uint32_t spins = 0;
            // relaxed polls (one acquire fence after the last flag): a poll is a plain L2 read of local memory
            while ((int32_t)(*((volatile const uint32_t*)(p.tp.flags_local + q * TP_FLAG_STRIDE + c)) - e) < 0) {
              if ((++spins & 15u) == 0u) {
                if (*abort_flag || *((volatile uint32_t*)p.status) != PG_ST_OK) {
                  *abort_flag = 1;
                  w_ok = false;
                  break;
                }
                if (globaltimer_ns() - t0 > p.tp.wait_ns) {
                  atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | ((50u + (uint32_t)ph) << 8) | ((uint32_t)q << 16));
                  *abort_flag = 1;
                  w_ok = false;
                  break;
                }
              }
            }
          }
          asm volatile("fence.acq_rel.sys;" ::: "memory");
          if (ts) ts[15] = globaltimer_ns();  // every rank's partial of these units has arrived
          ok = w_ok;
        }
        ok = bar128(ok);
        if (ok) {
          const bf16* y_mc = p.tp.y_mc[par];
          for (int u = c * EW + ew; u < units; u += 2 * EW * G) {
            // both units' sums over the ranks are requested from the switch before either is used
            const int uu[2] = {u, u + EW * G};
            FixIn f[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              f[k].part = 0.f;
              f[k].a = make_float4(0.f, 0.f, 0.f, 0.f);
              f[k].rv = make_uint2(0u, 0u);
              f[k].wv = make_uint2(0u, 0u);
              const int rt = uu[k] / p.T, n = uu[k] - rt * p.T;
              const int mcol = (rem0 + rt) * BM + lane * 4;
              if (uu[k] < units && mcol + 3 < P.M) {
                const size_t off = (size_t)n * P.M + mcol;
                if (p.tp.use_multimem) {
                  const uint2 sum = multimem_ld_reduce_bf16x4(y_mc + off);
                  const float2 s0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&sum.x)), s1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&sum.y));
                  f[k].a = make_float4(s0.x, s0.y, s1.x, s1.y);
                } else {
                  // every rank's copy over NVLink, all loads in flight, added in rank order (the same order on every rank)
                  uint2 part[TP_MAX_RANKS];
#pragma unroll
                  for (int q = 0; q < TP_MAX_RANKS; ++q)
                    part[q] = q < p.tp.world ? ld_relaxed_sys_u32x2(p.tp.y_peer[q][par] + off) : make_uint2(0u, 0u);
#pragma unroll
                  for (int q = 0; q < TP_MAX_RANKS; ++q) {
                    if (q < p.tp.world) {
                      const float2 s0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&part[q].x)), s1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&part[q].y));
                      f[k].a.x += s0.x;
                      f[k].a.y += s0.y;
                      f[k].a.z += s1.x;
                      f[k].a.w += s1.y;
                    }
                  }
                }
                f[k].rv = __ldcg(reinterpret_cast<const uint2*>(p.residual + (size_t)n * p.ld_res + mcol));
                f[k].wv = *reinterpret_cast<const uint2*>(P.norm_w + mcol);
              }
            }
            fix_finish(p, P, uu[0], rem0, lane, f[0], false);
            if (uu[1] < units) fix_finish(p, P, uu[1], rem0, lane, f[1], false);
          }
        }
        ++tp_sites;
      } else if (ok && need_fix) {
        // units (remainder tile, token): one warp each, a lane finishes 4 consecutive weight rows.  Two
        // units are in flight per warp: all loads of both are issued before the first value is used.
        const int units = P.rem_tiles * p.T;
        for (int u = c * EW + ew; u < units; u += 2 * EW * G) {
          const int u2 = u + EW * G;
          const bool two = u2 < units;
          FixIn f1, f2;
          fix_load(p, P, u, rem0, lane, f1);
          if (two) fix_load(p, P, u2, rem0, lane, f2);
          fix_finish(p, P, u, rem0, lane, f1);
          if (two) fix_finish(p, P, u2, rem0, lane, f2);
        }
      }
      // ---- the phase's output is complete on this CTA: second grid barrier ----
      ok = bar128(ok);
      if (ts) ts[4 + 3 * ph] = globaltimer_ns();  // fix-up of this CTA done
      if (et == 0) grid_arrive(bar_b);
      if (!ok) break;
    }
    // last CTA through re-arms the counters for the next launch (every CTA is past every wait by then:
    // a CTA arrives here only after it passed all of them)
    if (et == 0) {
      uint32_t* fin = p.counters + 3 * MAX_PHASES;
      __threadfence();
      const uint32_t old = atomicAdd(fin, 1u);
      if (old == (uint32_t)G - 1u) {
        // nobody waits on `fin`; the token producers of other CTAs may still poll the last bar_b only if a
        // later phase existed, which it does not
        for (int i = 0; i <= 3 * MAX_PHASES; ++i) p.counters[i] = 0u;
        if (p.tp.world > 1) *p.tp.epoch = tp_epoch + (uint32_t)tp_sites;  // the next launch numbers its exchanges from here
        __threadfence();
      }
    }
  }
  if (*abort_flag) {
    // a wait gave up: bulk copies of this CTA may still be in flight; give them time to land in this
    // CTA's shared memory before it is handed to another CTA
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (9u << 8));
}

std::mutex g_mu;
unsigned long long* g_chain_timing = nullptr;
bool g_attr[64];
int g_sms[64];
int g_smem[64];

}  // namespace

// One descriptor per GEMM phase of pg_decode_chain.
struct PgChainPhase {
  const void* x;      // [T, K] bf16 input rows of the phase (phase 0: caller's input; later: the previous phase's `out`)
  long long ldx;
  const void* w;      // [M, K] bf16
  long long ldw;
  int M, K;
  int epi;            // 0 plain, 1 SwiGLU over interleaved (gate, up) rows (out is [T, M / 2]), 2 residual add + norm-weight product (out = h * norm_w, RMSNorm scale owed: out_ssp)
  void* out;
  long long ld_out;
  const void* norm_w;  // epi 2
  int norm_offset;
  const void* in_ssp;  // sums of squares owed by the input rows ([T][in_ld] f32, in_parts valid per row, in_width = normalised width); NULL = input is final
  int in_parts, in_ld, in_width;
  float in_eps;
  void* out_ssp;       // epi 2: [T][out_ld] f32, entry [token][weight tile]
  int out_ld;
  // epi 3 (fused qkv rows [q heads | k heads | v heads], head_dim 128): per-head RMSNorm (q_w / k_w, NULL = none; norm_offset = (1 + w)),
  // rotary embedding from cos / sin [max_pos][rot / 2] at positions[T], q to `out` [T, hq, 128], k / v into kv [pages, 2, page_size, hkv, 128] at slots[T]
  const void* q_w;
  const void* k_w;
  const void* cos;
  const void* sin;
  const void* positions;
  const void* slots;
  void* kv;
  int hq, hkv, rot, page_size, max_pos;
  long long num_slots;
  float qk_eps;
};

// Profiling hook: a device buffer of 16 x uint64 per CTA that every following launch fills with
// globaltimer stamps: [0] entry, [1] predecessor complete, then per phase p: [2 + 3p] this CTA's tiles
// stored, [3 + 3p] all CTAs' partials visible, [4 + 3p] this CTA's fix-up done.  nullptr = off.
extern "C" void pg_decode_chain_set_timing(void* buf) { g_chain_timing = (unsigned long long*)buf; }

extern "C" long long pg_decode_chain_ws_bytes(int device) {
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
  return (long long)sms * 2 * SLOT_FLOATS * 4;
}

// Runs `nphase` (1..4) dependent GEMMs for a decode step of T <= 64 rows in one launch.
// `residual` [T, hidden] is updated in place by every epi-2 phase.  `ws` holds
// pg_decode_chain_ws_bytes() bytes; `counters` holds 16 uint32 that are zero before the first
// launch (every completed launch leaves them zero).
// Tensor-parallel description for pg_decode_chain_tp: `y_local` / `y_mc` are this rank's two partial buffers
// (each at least 64 x max M bf16) and the same buffers through the multicast mapping; `flags_peer[q]` is rank
// q's flag block (8 x 160 uint32 arrival words, one per source rank and CTA, + the exchange counter at word 1280; 8 KiB, all zero at start), `flags_peer[rank]`
// the local one.
struct PgChainTp {
  int world, rank;
  void* y_local[2];
  const void* y_mc[2];
  void* flags_peer[8];
  unsigned long long wait_ns;
  const void* y_peer[8][2];  // every rank's two partial buffers (peer mapped; [rank] = y_local)
  int use_multimem;          // 1: multimem.ld_reduce; 0: plain peer loads added in rank order
};

static int decode_chain_impl(const PgChainPhase* phases, int nphase, int T, void* residual, long long ld_res, float eps, void* ws, long long ws_bytes, void* counters,
                             void* status, const PgChainTp* tp, cudaStream_t stream);

extern "C" int pg_decode_chain(const PgChainPhase* phases, int nphase, int T, void* residual, long long ld_res, float eps, void* ws, long long ws_bytes,
                               void* counters, void* status, cudaStream_t stream) {
  return decode_chain_impl(phases, nphase, T, residual, ld_res, eps, ws, ws_bytes, counters, status, nullptr, stream);
}

// The same chain on one rank of a tensor-parallel group: every residual + norm phase sums its result over the
// ranks through NVSwitch multicast memory (see ChainTp).  All ranks must launch the same sequence of chains.
extern "C" int pg_decode_chain_tp(const PgChainPhase* phases, int nphase, int T, void* residual, long long ld_res, float eps, void* ws, long long ws_bytes,
                                  void* counters, void* status, const PgChainTp* tp, cudaStream_t stream) {
  PG_REQUIRE(tp != nullptr && tp->world >= 2 && tp->world <= TP_MAX_RANKS && tp->rank >= 0 && tp->rank < tp->world, "decode chain: bad tensor-parallel description");
  for (int i = 0; i < 2; ++i) PG_REQUIRE(tp->y_local[i] && tp->y_mc[i] && ((uintptr_t)tp->y_local[i] & 15) == 0 && ((uintptr_t)tp->y_mc[i] & 15) == 0, "decode chain: partial buffers must be given and 16-byte aligned");
  for (int q = 0; q < tp->world; ++q) PG_REQUIRE(tp->flags_peer[q] != nullptr, "decode chain: flag block of rank %d is missing", q);
  return decode_chain_impl(phases, nphase, T, residual, ld_res, eps, ws, ws_bytes, counters, status, tp, stream);
}

static int decode_chain_impl(const PgChainPhase* phases, int nphase, int T, void* residual, long long ld_res, float eps, void* ws, long long ws_bytes, void* counters,
                             void* status, const PgChainTp* tp, cudaStream_t stream) {
  PG_REQUIRE(nphase >= 1 && nphase <= MAX_PHASES, "decode chain: %d phases (1..%d)", nphase, MAX_PHASES);
  PG_REQUIRE(T >= 1 && T <= BN, "decode chain: built for steps of 1..%d token rows, got %d", BN, T);
  PG_REQUIRE(status != nullptr && counters != nullptr && ws != nullptr, "decode chain: scratch, counters and status word are required");
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_attr[dev & 63]) {
      PG_CUDA(cudaDeviceGetAttribute(&g_sms[dev & 63], cudaDevAttrMultiProcessorCount, dev));
      PG_CUDA(cudaDeviceGetAttribute(&g_smem[dev & 63], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      PG_CUDA(cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_smem[dev & 63]));
      g_attr[dev & 63] = true;
    }
  }
  const int G = g_sms[dev & 63];
  PG_REQUIRE(ws_bytes >= (long long)G * 2 * SLOT_FLOATS * 4, "decode chain: scratch too small");
  const size_t smem = 1024 + (size_t)NW * W_BYTES + (size_t)NX * X_BYTES + (2 * NW + 2 * NX + 4) * 8 + 16 + BN * 4;
  PG_REQUIRE((int)smem <= g_smem[dev & 63], "decode chain: needs %zu bytes of shared memory", smem);
  ChainParams p;
  memset(&p, 0, sizeof(p));
  TMaps tm;
  memset(&tm, 0, sizeof(tm));
  p.nphase = nphase;
  p.T = T;
  p.G = G;
  p.residual = (bf16*)residual;
  p.ld_res = ld_res;
  p.eps = eps;
  p.ws = (float*)ws;
  p.counters = (uint32_t*)counters;
  p.status = (uint32_t*)status;
  p.timing = g_chain_timing;
  if (tp) {
    p.tp.world = tp->world;
    p.tp.rank = tp->rank;
    for (int i = 0; i < 2; ++i) {
      p.tp.y_local[i] = (bf16*)tp->y_local[i];
      p.tp.y_mc[i] = (const bf16*)tp->y_mc[i];
    }
    for (int q = 0; q < tp->world; ++q) {
      p.tp.flags_peer[q] = (uint32_t*)tp->flags_peer[q];
      for (int i = 0; i < 2; ++i) {
        p.tp.y_peer[q][i] = (const bf16*)tp->y_peer[q][i];
        PG_REQUIRE(tp->use_multimem || tp->y_peer[q][i] != nullptr, "decode chain: partial buffer %d of rank %d is missing", i, q);
      }
    }
    p.tp.use_multimem = tp->use_multimem;
    p.tp.flags_local = (uint32_t*)tp->flags_peer[tp->rank];
    p.tp.epoch = p.tp.flags_local + TP_EPOCH_WORD;
    PG_REQUIRE(G <= TP_FLAG_STRIDE, "decode chain: %d SMs exceed the per-rank flag stride", G);
    p.tp.wait_ns = tp->wait_ns ? tp->wait_ns : PG_WAIT_LIMIT_NS;
  }
  for (int i = 0; i < nphase; ++i) {
    const PgChainPhase& s = phases[i];
    Phase& P = p.ph[i];
    PG_REQUIRE(s.M > 0 && s.K > 0 && s.K % 8 == 0, "decode chain: phase %d has M=%d K=%d (K must be a multiple of 8)", i, s.M, s.K);
    PG_REQUIRE(s.epi >= CH_PLAIN && s.epi <= CH_QKV_ROPE, "decode chain: phase %d has unknown epilogue %d", i, s.epi);
    P.M = s.M;
    P.K = s.K;
    P.kblocks = ceil_div(s.K, BK);
    P.tiles = ceil_div(s.M, BM);
    P.full_rounds = P.tiles / G;
    P.rem_tiles = P.tiles - P.full_rounds * G;
    PG_REQUIRE((long long)P.rem_tiles * P.kblocks < (1ll << 30), "decode chain: phase %d is too large", i);
    P.per_cta = P.rem_tiles ? (P.rem_tiles * P.kblocks + G - 1) / G : 0;
    P.epi = s.epi;
    P.out = (bf16*)s.out;
    P.ld_out = s.ld_out;
    P.norm_w = (const bf16*)s.norm_w;
    P.norm_offset = s.norm_offset;
    P.in_ssp = (const float*)s.in_ssp;
    P.in_parts = s.in_parts;
    P.in_ld = s.in_ld;
    P.in_width = s.in_width;
    P.in_eps = s.in_eps;
    P.out_ssp = (float*)s.out_ssp;
    P.out_ld = s.out_ld;
    PG_REQUIRE(s.in_ssp == nullptr || (s.in_parts > 0 && s.in_ld >= s.in_parts && s.in_width > 0), "decode chain: phase %d has an incomplete input-scale description", i);
    if (s.epi == CH_QKV_ROPE) {
      PG_REQUIRE(P.full_rounds == 0 && s.M == (s.hq + 2 * s.hkv) * BM, "decode chain: the qkv + RoPE phase needs head_dim %d and M = (hq + 2 hkv) * %d < %d * %d rows", BM, BM, G, BM);
      PG_REQUIRE(s.rot % 2 == 0 && s.rot <= BM && s.cos && s.sin && s.positions && s.slots && s.kv && s.out && s.page_size > 0,
                 "decode chain: the qkv + RoPE phase needs rotary tables, positions, slots, the KV page buffer and the q output");
      PG_REQUIRE(s.rot == BM || s.rot == 0, "decode chain: the fused RoPE rotates the whole 128-wide head (rotary dim %d)", s.rot);
      PG_REQUIRE((s.q_w == nullptr) == (s.k_w == nullptr), "decode chain: q and k norm weights come together");
      P.q_w = (const bf16*)s.q_w;
      P.k_w = (const bf16*)s.k_w;
      P.has_qk_norm = s.q_w != nullptr;
      P.cos = (const bf16*)s.cos;
      P.sin = (const bf16*)s.sin;
      P.positions = (const int*)s.positions;
      P.slots = (const int*)s.slots;
      P.kv = (bf16*)s.kv;
      P.hq = s.hq;
      P.hkv = s.hkv;
      P.rot = s.rot;
      P.page_size = s.page_size;
      P.max_pos = s.max_pos;
      P.num_slots = s.num_slots;
      P.qk_eps = s.qk_eps;
    }
    if (s.epi == CH_SWIGLU) PG_REQUIRE(s.M % 4 == 0 && s.ld_out % 2 == 0 && ((uintptr_t)s.out & 3) == 0, "decode chain: SwiGLU phase needs M %% 4 == 0 and a 4-byte aligned output");
    if (s.epi == CH_PLAIN) PG_REQUIRE(s.M % 4 == 0 && s.ld_out % 4 == 0 && ((uintptr_t)s.out & 7) == 0, "decode chain: plain phase needs M %% 4 == 0 and an 8-byte aligned output");
    if (s.epi == CH_RESID_NORM) {
      PG_REQUIRE(residual != nullptr && s.norm_w != nullptr && s.out_ssp != nullptr && s.out_ld >= ceil_div(s.M, BM), "decode chain: phase %d needs the residual, a norm weight and room for the sums of squares", i);
      PG_REQUIRE(P.full_rounds == 0 && s.M % BM == 0 && P.tiles <= 64, "decode chain: residual + norm phase needs M (%d) to be a multiple of %d, at most %d", s.M, BM, 64 * BM);
      PG_REQUIRE(ld_res % 4 == 0 && s.ld_out % 4 == 0 && ((uintptr_t)residual & 7) == 0 && ((uintptr_t)s.out & 7) == 0 && ((uintptr_t)s.norm_w & 7) == 0,
                 "decode chain: residual, output and norm weight must be 8-byte aligned");
    }
    // a k-range never spans more than two tiles: per_cta <= kblocks because rem_tiles < G
    int rc = pg_make_tmap_bf16_2d(&tm.w[i], s.w, s.M, s.K, s.ldw, BM, BK);
    if (rc) return rc;
    rc = pg_make_tmap_bf16_2d(&tm.x[i], s.x, T, s.K, s.ldx, BN, BK);
    if (rc) return rc;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)G);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1u : 0u;
  PG_CUDA(cudaLaunchKernelEx(&cfg, decode_chain_kernel, tm, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
