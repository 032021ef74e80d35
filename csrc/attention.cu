// Paged GQA attention (bf16, head_dim 64/128/256, page size 16/32/64).
//
// Decode (one query row per sequence): split-KV flash decoding.  A CTA owns one
// (sequence, kv head, split); its warps stride over 16-token KV tiles, each warp with
// its own cp.async pipeline and online-softmax state, so the main loop has no
// CTA-wide barrier.  The GQA group's query heads are the (zero-padded) 16 rows of the
// MMA A operand; K is the B operand straight from the swizzled page tile, P is reused
// from the S accumulators as the A operand of P*V.  Warps merge through shared memory;
// splits merge in a second small kernel (deterministic order).  Padding sequences
// (kv_len == 0) produce zeros, which keeps CUDA-graph buckets inert.
//
// Prefill / mixed (ragged query rows, causal): a CTA owns 64 query rows of one query
// head (4 warps x 16 rows) and walks 64-token KV tiles through a double-buffered
// cp.async pipeline.
//
// Tensor work here runs on warp-level mma.sync: at head_dim 128 decode attention is
// bound by KV bytes, not tensor throughput.  KV layout per layer:
// [pages, 2, page_size, kv_heads, head_dim].
//
// Takes the place of the reference's FlashInfer instantiations
// (pegainfer-kernels/csrc/shared/paged_attention.cu:85-279 decode/split-KV, :455-620
// batch prefill, :977-1135 head_dim 256).
#include <float.h>

#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
// Same, marked evict-first in L2: the KV cache is streamed once per step and must not push
// out lines that are about to be reused (prefetched weights of the next GEMM).
__device__ __forceinline__ void cp_async16_stream(void* dst, const void* src, bool valid, uint64_t policy) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr float NEG_BIG = -1e30f;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  const bf16* q;       // [T, Hq, D]
  const bf16* kv;      // [pages, 2, ps, Hkv, D]
  bf16* out;           // [T, Hq*D]
  const int* q_indptr; // [B+1]
  const int* kv_lens;  // [B]
  const int* table;    // [B, table_stride]
  int table_stride;
  int num_seqs, hq, hkv, page_size;
  float scale_log2;
  int splits;
  float* part_o;    // [B, Hq, splits, D]
  float* part_lse;  // [B, Hq, splits]
  long long num_pages;
  uint32_t* status;
  int window;  // decode: a row sees its last `window` keys only (0: all of them)
};

// Row address of token `tok` of sequence b, kv head h (kvsel 0 = K, 1 = V).
template <int D>
__device__ __forceinline__ const bf16* kv_row(const AttnParams& p, const int* table_row, int tok, int h, int kvsel) {
  const int page = table_row[tok / p.page_size];
  const int off = tok % p.page_size;
  return p.kv + ((((long long)page * 2 + kvsel) * p.page_size + off) * p.hkv + h) * D;
}

// Swizzled offset (in bf16 elements) of 16-byte chunk `ch` of row `r` in a [rows][D] tile.
template <int D>
__device__ __forceinline__ int swz(int r, int ch) {
  return r * D + ((ch ^ (r & 7)) << 3);
}

// -----------------------------------------------------------------------------------
// decode
// -----------------------------------------------------------------------------------
template <int D, int STAGES>
__global__ void __launch_bounds__(128, (STAGES == 2 && D <= 128) ? 3 : 1) decode_attn_kernel(const AttnParams p) {
  PG_PDL_ENTRY();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int TILE = 16;
  constexpr int CH = D / 8;            // 16-byte chunks per row
  constexpr int KS = D / 16;           // k-steps of Q*K^T
  constexpr int NT = D / 8;            // n-tiles of P*V
  constexpr int STAGE_ELEMS = 2 * TILE * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int split = blockIdx.x % p.splits;
  const int h = (blockIdx.x / p.splits) % p.hkv;
  const int b = blockIdx.x / (p.splits * p.hkv);
  const int G = p.hq / p.hkv;
  const int kv_len = p.kv_lens[b];
  const int qrow = p.q_indptr[b];
  const int* table_row = p.table + (long long)b * p.table_stride;
  bf16* wsm = reinterpret_cast<bf16*>(smem_raw) + warp * STAGES * STAGE_ELEMS;

  const int kv_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;  // first key the row (position kv_len - 1) may see
  const int first_tile = kv_lo / TILE;
  const int n_tiles = (kv_len + TILE - 1) / TILE - first_tile;
  const int tps = (n_tiles + p.splits - 1) / p.splits;
  const int t_begin = first_tile + split * tps;
  const int t_end = min(first_tile + n_tiles, t_begin + tps);

  // Q fragments: rows 0..G-1 of the A operand are the group's heads, the rest zero.
  uint32_t qf[KS][2];
  {
    const bf16* qh = p.q + ((long long)qrow * p.hq + (long long)h * G + g) * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      if (g < G) {
        qf[ks][0] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t4);
        qf[ks][1] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 8 + 2 * t4);
      } else {
        qf[ks][0] = 0u;
        qf[ks][1] = 0u;
      }
    }
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run = NEG_BIG, l_run = 0.f;

  // A 16-token tile never straddles a page (page sizes are multiples of 16): one table
  // lookup per tile, then plain strides.
  const long long row_stride = (long long)p.hkv * D;
  const long long v_plane = (long long)p.page_size * row_stride;
  const uint64_t kv_policy = l2_policy_evict_first();
  auto issue = [&](int tile, int stage) {
    bf16* ks_ = wsm + stage * STAGE_ELEMS;
    bf16* vs_ = ks_ + TILE * D;
    if (tile < t_end) {
      const int tok0 = tile * TILE;
      const int page = table_row[tok0 / p.page_size];
      const bf16* kbase = p.kv + ((long long)page * 2 * p.page_size + (tok0 % p.page_size)) * row_stride + (long long)h * D;
#pragma unroll
      for (int i = 0; i < (TILE * CH) / 32; ++i) {
        const int c = lane + 32 * i;
        const int r = c / CH, ch = c % CH;
        const bool valid = tok0 + r < kv_len;
        const bf16* src = kbase + (valid ? r : 0) * row_stride + ch * 8;
        cp_async16_stream(ks_ + swz<D>(r, ch), src, valid, kv_policy);
        cp_async16_stream(vs_ + swz<D>(r, ch), src + v_plane, valid, kv_policy);
      }
    }
    cp_async_commit();
  };

  const int first = t_begin + warp;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(first + s * 4, s);

  int it = 0;
  for (int tile = first; tile < t_end; tile += 4, ++it) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    issue(tile + (STAGES - 1) * 4, (it + STAGES - 1) % STAGES);
    const bf16* ks_ = wsm + (it % STAGES) * STAGE_ELEMS;
    const bf16* vs_ = ks_ + TILE * D;

    float s_acc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int j = lane >> 3, r = lane & 7;
      const int row = (j >> 1) * 8 + r;
      const int ch = ks * 2 + (j & 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(smem_u32(ks_ + swz<D>(row, ch)), b0, b1, b2, b3);
      const uint32_t a[4] = {qf[ks][0], 0u, qf[ks][1], 0u};
      mma16816(s_acc[0], a, b0, b1);
      mma16816(s_acc[1], a, b2, b3);
    }
    // online softmax for row g (rows g+8 are padding)
    float sv[4];
    const int tok0 = tile * TILE + 2 * t4;
    sv[0] = (tok0 < kv_len && tok0 >= kv_lo) ? s_acc[0][0] * p.scale_log2 : NEG_BIG;
    sv[1] = (tok0 + 1 < kv_len && tok0 + 1 >= kv_lo) ? s_acc[0][1] * p.scale_log2 : NEG_BIG;
    sv[2] = (tok0 + 8 < kv_len && tok0 + 8 >= kv_lo) ? s_acc[1][0] * p.scale_log2 : NEG_BIG;
    sv[3] = (tok0 + 9 < kv_len && tok0 + 9 >= kv_lo) ? s_acc[1][1] * p.scale_log2 : NEG_BIG;
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float corr = exp2f(m_run - m_new);
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pv[i] = sv[i] <= NEG_BIG ? 0.f : exp2f(sv[i] - m_new);
    float ps = pv[0] + pv[1] + pv[2] + pv[3];
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    l_run = l_run * corr + ps;
    m_run = m_new;
    const uint32_t pa[4] = {pack_bf16(pv[0], pv[1]), 0u, pack_bf16(pv[2], pv[3]), 0u};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= corr;
      o[n][1] *= corr;
    }
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      const int j = lane >> 3, r = lane & 7;
      const int row = (j & 1) * 8 + r;
      const int ch = n2 * 2 + (j >> 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(smem_u32(vs_ + swz<D>(row, ch)), b0, b1, b2, b3);
      mma16816(o[2 * n2], pa, b0, b1);
      mma16816(o[2 * n2 + 1], pa, b2, b3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps: [warp][row][D] f32 partials + (m, l)
  float* mo = reinterpret_cast<float*>(smem_raw);
  float* mm = mo + 4 * 8 * D;
  float* ml = mm + 4 * 8;
  if (g < 8) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mo[(warp * 8 + g) * D + n * 8 + 2 * t4] = o[n][0];
      mo[(warp * 8 + g) * D + n * 8 + 2 * t4 + 1] = o[n][1];
    }
    if (t4 == 0) {
      mm[warp * 8 + g] = m_run;
      ml[warp * 8 + g] = l_run;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += 128) {
    const int row = idx / D, d = idx % D;
    float M = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 8 + row]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(mm[w * 8 + row] - M);
      L += f * ml[w * 8 + row];
      O += f * mo[(w * 8 + row) * D + d];
    }
    const int hq = h * G + row;
    const float val = L > 0.f ? O / L : 0.f;
    if (p.splits == 1) {
      p.out[((long long)qrow * p.hq + hq) * D + d] = __float2bfloat16(val);
    } else {
      p.part_o[(((long long)b * p.hq + hq) * p.splits + split) * D + d] = val;
      if (d == 0) p.part_lse[((long long)b * p.hq + hq) * p.splits + split] = L > 0.f ? M + log2f(L) : NEG_BIG;
    }
  }
}

// -----------------------------------------------------------------------------------
// decode, persistent form
// -----------------------------------------------------------------------------------
// One work unit = (sequence, kv head, KV split), as above, but the grid is one CTA per
// resident slot and every CTA walks units blockIdx.x, blockIdx.x + gridDim.x, ...  Each
// warp treats its share of the tiles of all those units as ONE stream: the cp.async issue
// cursor runs two tiles ahead of the compute cursor across unit boundaries, so the pipeline
// is filled once per CTA instead of once per unit (a unit is only a handful of tiles per
// warp, and a pipeline that covers DRAM latency takes about as long to fill).  The merge
// scratch is separate from the pipeline buffers, because loads of the next unit are in
// flight while the four warps of a CTA combine their partials of the current one.
struct DecodeUnit {
  int b, h, split, kv_len, kv_lo, qrow, t_begin, t_end;
  const int* table_row;
};

__device__ __forceinline__ bool load_decode_unit(const AttnParams& p, int u, DecodeUnit& o) {
  if (u >= p.num_seqs * p.hkv * p.splits) return false;
  o.split = u % p.splits;
  o.h = (u / p.splits) % p.hkv;
  o.b = u / (p.splits * p.hkv);
  o.kv_len = p.kv_lens[o.b];
  o.qrow = p.q_indptr[o.b];
  o.table_row = p.table + (long long)o.b * p.table_stride;
  o.kv_lo = p.window > 0 ? max(0, o.kv_len - p.window) : 0;  // first key the row (position kv_len - 1) may see
  const int first_tile = o.kv_lo / 16;
  const int n_tiles = (o.kv_len + 15) / 16 - first_tile;
  const int tps = (n_tiles + p.splits - 1) / p.splits;
  o.t_begin = first_tile + o.split * tps;
  o.t_end = min(first_tile + n_tiles, o.t_begin + tps);
  return true;
}

template <int D>
__global__ void __launch_bounds__(128, D <= 128 ? 2 : 1) decode_attn_persistent_kernel(const AttnParams p) {
  PG_PDL_ENTRY();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int STAGES = 3;
  constexpr int TILE = 16;
  constexpr int CH = D / 8;
  constexpr int KS = D / 16;
  constexpr int NT = D / 8;
  constexpr int STAGE_ELEMS = 2 * TILE * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = p.hq / p.hkv;
  bf16* wsm = reinterpret_cast<bf16*>(smem_raw) + warp * STAGES * STAGE_ELEMS;
  // merge scratch behind the pipelines: [warp][8 rows][D] f32 + (m, l) per warp and row
  float* mo = reinterpret_cast<float*>(smem_raw + (size_t)4 * STAGES * STAGE_ELEMS * 2);
  float* mm = mo + 4 * 8 * D;
  float* ml = mm + 4 * 8;
  const long long row_stride = (long long)p.hkv * D;
  const long long v_plane = (long long)p.page_size * row_stride;
  const uint64_t kv_policy = l2_policy_evict_first();

  // issue cursor
  DecodeUnit ui;
  int iu = blockIdx.x;
  bool vi = load_decode_unit(p, iu, ui);
  int ti = vi ? ui.t_begin + warp : 0;
  auto issue_next = [&](int stage) {
    while (vi && ti >= ui.t_end) {
      iu += gridDim.x;
      vi = load_decode_unit(p, iu, ui);
      ti = vi ? ui.t_begin + warp : 0;
    }
    if (vi) {
      bf16* ks_ = wsm + stage * STAGE_ELEMS;
      bf16* vs_ = ks_ + TILE * D;
      const int tok0 = ti * TILE;
      const int page = ui.table_row[tok0 / p.page_size];
      const bf16* kbase = p.kv + ((long long)page * 2 * p.page_size + (tok0 % p.page_size)) * row_stride + (long long)ui.h * D;
#pragma unroll
      for (int i = 0; i < (TILE * CH) / 32; ++i) {
        const int c = lane + 32 * i;
        const int r = c / CH, ch = c % CH;
        const bool valid = tok0 + r < ui.kv_len;
        const bf16* src = kbase + (valid ? r : 0) * row_stride + ch * 8;
        cp_async16_stream(ks_ + swz<D>(r, ch), src, valid, kv_policy);
        cp_async16_stream(vs_ + swz<D>(r, ch), src + v_plane, valid, kv_policy);
      }
      ti += 4;
    }
    cp_async_commit();  // one group per call, also when nothing was left to load
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue_next(s);

  // compute cursor
  DecodeUnit uc;
  int cu = blockIdx.x;
  bool vc = load_decode_unit(p, cu, uc);
  int it = 0;
  while (vc) {
    uint32_t qf[KS][2];
    {
      const bf16* qh = p.q + ((long long)uc.qrow * p.hq + (long long)uc.h * G + g) * D;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        if (g < G) {
          qf[ks][0] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t4);
          qf[ks][1] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 8 + 2 * t4);
        } else {
          qf[ks][0] = 0u;
          qf[ks][1] = 0u;
        }
      }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run = NEG_BIG, l_run = 0.f;
    for (int tile = uc.t_begin + warp; tile < uc.t_end; tile += 4, ++it) {
      cp_async_wait<STAGES - 2>();
      __syncwarp();
      issue_next((it + STAGES - 1) % STAGES);
      const bf16* ks_ = wsm + (it % STAGES) * STAGE_ELEMS;
      const bf16* vs_ = ks_ + TILE * D;
      float s_acc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int j = lane >> 3, r = lane & 7;
        const int row = (j >> 1) * 8 + r;
        const int ch = ks * 2 + (j & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(ks_ + swz<D>(row, ch)), b0, b1, b2, b3);
        const uint32_t a[4] = {qf[ks][0], 0u, qf[ks][1], 0u};
        mma16816(s_acc[0], a, b0, b1);
        mma16816(s_acc[1], a, b2, b3);
      }
      float sv[4];
      const int tok0 = tile * TILE + 2 * t4;
      sv[0] = (tok0 < uc.kv_len && tok0 >= uc.kv_lo) ? s_acc[0][0] * p.scale_log2 : NEG_BIG;
      sv[1] = (tok0 + 1 < uc.kv_len && tok0 + 1 >= uc.kv_lo) ? s_acc[0][1] * p.scale_log2 : NEG_BIG;
      sv[2] = (tok0 + 8 < uc.kv_len && tok0 + 8 >= uc.kv_lo) ? s_acc[1][0] * p.scale_log2 : NEG_BIG;
      sv[3] = (tok0 + 9 < uc.kv_len && tok0 + 9 >= uc.kv_lo) ? s_acc[1][1] * p.scale_log2 : NEG_BIG;
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float corr = exp2f(m_run - m_new);
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = sv[i] <= NEG_BIG ? 0.f : exp2f(sv[i] - m_new);
      float ps = pv[0] + pv[1] + pv[2] + pv[3];
      ps += __shfl_xor_sync(0xffffffffu, ps, 1);
      ps += __shfl_xor_sync(0xffffffffu, ps, 2);
      l_run = l_run * corr + ps;
      m_run = m_new;
      const uint32_t pa[4] = {pack_bf16(pv[0], pv[1]), 0u, pack_bf16(pv[2], pv[3]), 0u};
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][0] *= corr;
        o[n][1] *= corr;
      }
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = (j & 1) * 8 + r;
        const int ch = n2 * 2 + (j >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vs_ + swz<D>(row, ch)), b0, b1, b2, b3);
        mma16816(o[2 * n2], pa, b0, b1);
        mma16816(o[2 * n2 + 1], pa, b2, b3);
      }
    }
    // unit done for this warp: combine the four warps (the next unit's loads stay in flight)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mo[(warp * 8 + g) * D + n * 8 + 2 * t4] = o[n][0];
      mo[(warp * 8 + g) * D + n * 8 + 2 * t4 + 1] = o[n][1];
    }
    if (t4 == 0) {
      mm[warp * 8 + g] = m_run;
      ml[warp * 8 + g] = l_run;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += 128) {
      const int row = idx / D, d = idx % D;
      float M = NEG_BIG;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 8 + row]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(mm[w * 8 + row] - M);
        L += f * ml[w * 8 + row];
        O += f * mo[(w * 8 + row) * D + d];
      }
      const int hq = uc.h * G + row;
      const float val = L > 0.f ? O / L : 0.f;
      if (p.splits == 1) {
        p.out[((long long)uc.qrow * p.hq + hq) * D + d] = __float2bfloat16(val);
      } else {
        p.part_o[(((long long)uc.b * p.hq + hq) * p.splits + uc.split) * D + d] = val;
        if (d == 0) p.part_lse[((long long)uc.b * p.hq + hq) * p.splits + uc.split] = L > 0.f ? M + log2f(L) : NEG_BIG;
      }
    }
    __syncthreads();  // the scratch is free again
    cu += gridDim.x;
    vc = load_decode_unit(p, cu, uc);
  }
  cp_async_wait<0>();
}

template <int D>
__global__ void __launch_bounds__(128) decode_merge_kernel(const AttnParams p) {
  PG_PDL_ENTRY();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;  // (b, hq)
  if (unit >= (long long)p.num_seqs * p.hq) return;
  const int b = (int)(unit / p.hq), hq = (int)(unit % p.hq);
  const float* lse = p.part_lse + unit * p.splits;
  float M = NEG_BIG;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, lse[s]);
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  float W = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float l = lse[s];
    if (l <= NEG_BIG) continue;
    const float f = exp2f(l - M);
    W += f;
    const float* po = p.part_o + (unit * p.splits + s) * D;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += f * po[lane + 32 * i];
  }
  const int qrow = p.q_indptr[b];
  bf16* out = p.out + ((long long)qrow * p.hq + hq) * D;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) out[lane + 32 * i] = __float2bfloat16(W > 0.f ? acc[i] / W : 0.f);
}

// -----------------------------------------------------------------------------------
// prefill / mixed
// -----------------------------------------------------------------------------------
// MINB: CTAs per SM the register allocation aims for (3 costs a few spilled words at D = 128).
template <int D, int MINB>
__global__ void __launch_bounds__(128, MINB) prefill_attn_kernel(const AttnParams p, int window) {
  PG_PDL_ENTRY();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int BQ = 64, BKV = 64;
  constexpr int CH = D / 8, KS = D / 16, NT = D / 8;
  constexpr int TILE_ELEMS = BKV * D;
  bf16* sm = reinterpret_cast<bf16*>(smem_raw);  // [2 stages][K|V][64][D], Q tile staged in stage 0 first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int hq = blockIdx.y;
  const int G = p.hq / p.hkv;
  const int h = hq / G;

  // locate (sequence, q tile) for this CTA
  int b = 0, tile_in_seq = 0;
  {
    // late query tiles attend to the most keys: hand them out first so the long CTAs do not form the tail
    int rem = (int)gridDim.x - 1 - (int)blockIdx.x;
    for (; b < p.num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + BQ - 1) / BQ;
      if (rem < nt) {
        tile_in_seq = rem;
        break;
      }
      rem -= nt;
    }
    if (b >= p.num_seqs) return;
  }
  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int* table_row = p.table + (long long)b * p.table_stride;
  const int row_base = tile_in_seq * BQ;           // first query row of this CTA within the sequence
  const int rows_here = min(BQ, q_len - row_base);
  const int pos_base = kv_len - q_len + row_base;  // absolute position of that row
  if (kv_len == 0) {
    for (int idx = threadIdx.x; idx < rows_here * D; idx += 128)
      p.out[((long long)(q0 + row_base + idx / D) * p.hq + hq) * D + idx % D] = __float2bfloat16(0.f);
    return;
  }

  // stage Q tile [64][D] into shared memory (swizzled), then into A fragments
  for (int c = threadIdx.x; c < BQ * CH; c += 128) {
    const int r = c / CH, ch = c % CH;
    const bool valid = r < rows_here;
    const bf16* src = p.q + ((long long)(q0 + row_base + (valid ? r : 0)) * p.hq + hq) * D + ch * 8;
    cp_async16(sm + swz<D>(r, ch), src, valid);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int j = lane >> 3, r = lane & 7;
    const int row = warp * 16 + (j & 1) * 8 + r;
    const int ch = ks * 2 + (j >> 1);
    ldsm_x4(smem_u32(sm + swz<D>(row, ch)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }
  __syncthreads();

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};

  const int max_pos = pos_base + rows_here - 1;  // last position any row of this CTA may attend to
  int kv_start = 0;
  if (window > 0) kv_start = max(0, pos_base - window + 1) / BKV * BKV;
  const int kv_end = min(kv_len, max_pos + 1);
  const int n_kv_tiles = (kv_end - kv_start + BKV - 1) / BKV;

  // A thread copies the same 16-byte chunk `ch` of RPT rows of every K and V tile.  Tiles start at
  // multiples of 64 tokens and pages hold 16, 32 or 64, so a tile spans at most four pages: their
  // table entries are read once per tile and the row addresses follow by shifts (a table lookup and
  // a division per chunk made address generation the larger part of this kernel's instructions).
  constexpr int RPT = BKV * CH / 128, RSTEP = 128 / CH;
  const int ps_shift = __ffs(p.page_size) - 1;
  const long long row_stride = (long long)p.hkv * D;
  const long long v_plane = (long long)p.page_size * row_stride;
  const int my_ch = threadIdx.x % CH, my_r0 = threadIdx.x / CH;
  const bf16* kv_head = p.kv + (long long)h * D + my_ch * 8;
  auto issue = [&](int kt, int stage) {
    bf16* ks_ = sm + stage * 2 * TILE_ELEMS;
    bf16* vs_ = ks_ + TILE_ELEMS;
    if (kt < n_kv_tiles) {
      const int tok_base = kv_start + kt * BKV;
      const int pg_first = tok_base >> ps_shift;
      int pg[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pg[j] = (j << ps_shift) < BKV ? table_row[min(pg_first + j, p.table_stride - 1)] : 0;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int r = my_r0 + i * RSTEP;
        const bool valid = tok_base + r < kv_end;
        const int rr = valid ? r : 0;
        const int j = rr >> ps_shift;
        const int page = j == 0 ? pg[0] : j == 1 ? pg[1] : j == 2 ? pg[2] : pg[3];
        const bf16* src = kv_head + ((long long)page * 2 * p.page_size + (rr & (p.page_size - 1))) * row_stride;
        cp_async16(ks_ + swz<D>(r, my_ch), src, valid);
        cp_async16(vs_ + swz<D>(r, my_ch), src + v_plane, valid);
      }
    }
    cp_async_commit();
  };

  issue(0, 0);
  const int qpos0 = pos_base + warp * 16 + g;  // position of this lane's row g; row g+8 is +8
  for (int kt = 0; kt < n_kv_tiles; ++kt) {
    issue(kt + 1, (kt + 1) & 1);
    cp_async_wait<1>();
    __syncthreads();
    const bf16* ks_ = sm + (kt & 1) * 2 * TILE_ELEMS;
    const bf16* vs_ = ks_ + TILE_ELEMS;
    const int tok_base = kv_start + kt * BKV;
    // warps whose 16 rows are all padding or all masked for this tile still take part in the barriers
    float s_acc[BKV / 8][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < BKV / 16; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = n2 * 16 + (j >> 1) * 8 + r;
        const int ch = ks * 2 + (j & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(ks_ + swz<D>(row, ch)), b0, b1, b2, b3);
        mma16816(s_acc[2 * n2], qf[ks], b0, b1);
        mma16816(s_acc[2 * n2 + 1], qf[ks], b2, b3);
      }
    }
    float mx[2] = {NEG_BIG, NEG_BIG};
    // every key of the tile is visible to every row of this warp (all but the tiles on the
    // diagonal of a causal prompt): no per-element position tests
    const bool full_tile = window <= 0 && tok_base + BKV - 1 <= pos_base + warp * 16 && tok_base + BKV <= kv_end;
    if (full_tile) {
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = s_acc[n][e] * p.scale_log2;
          s_acc[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok_base + n * 8 + 2 * t4 + (e & 1);
          const int qp = qpos0 + (e >> 1) * 8;
          bool ok = tok <= qp && tok < kv_end;
          if (window > 0) ok = ok && tok > qp - window;
          const float v = ok ? s_acc[n][e] * p.scale_log2 : NEG_BIG;
          s_acc[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
    }
    float corr[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float m_new = fmaxf(m_run[rr], mx[rr]);
      corr[rr] = exp2f(m_run[rr] - m_new);
      m_run[rr] = m_new;
    }
    float ps[2] = {0.f, 0.f};
    uint32_t pa[BKV / 16][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) {
      float pvv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pvv[e] = s_acc[n][e] <= NEG_BIG ? 0.f : exp2f(s_acc[n][e] - m_run[e >> 1]);
        ps[e >> 1] += pvv[e];
      }
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(pvv[0], pvv[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(pvv[2], pvv[3]);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 1);
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 2);
      l_run[rr] = l_run[rr] * corr[rr] + ps[rr];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = kk * 16 + (j & 1) * 8 + r;
        const int ch = n2 * 2 + (j >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vs_ + swz<D>(row, ch)), b0, b1, b2, b3);
        mma16816(o[2 * n2], pa[kk], b0, b1);
        mma16816(o[2 * n2 + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = warp * 16 + g + rr * 8;
    if (r < rows_here) {
      const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
      bf16* dst = p.out + ((long long)(q0 + row_base + r) * p.hq + hq) * D;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
      }
    }
  }
}

int g_decode_stages = 3;

template <int D, int STAGES>
int launch_decode_s(const AttnParams& p, cudaStream_t stream) {
  const size_t pipe = (size_t)4 * STAGES * 2 * 16 * D * 2;
  const size_t merge = (size_t)(4 * 8 * D + 64) * 4;
  const size_t smem = pipe > merge ? pipe : merge;
  static bool set = false;
  if (!set) {
    PG_CUDA(cudaFuncSetAttribute(decode_attn_kernel<D, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  PG_CUDA(launch_pdl(decode_attn_kernel<D, STAGES>, dim3(p.num_seqs * p.hkv * p.splits), dim3(128), (size_t)(smem), stream, p));
  PG_LAUNCH_CHECK();
  if (p.splits > 1) {
    PG_CUDA(launch_pdl(decode_merge_kernel<D>, dim3((p.num_seqs * p.hq + 3) / 4), dim3(128), (size_t)(0), stream, p));
    PG_LAUNCH_CHECK();
  }
  return PG_OK;
}

int g_decode_persistent = -1;  // PEGAINFER_ATTN_PERSISTENT=0 selects the one-unit-per-CTA kernel

template <int D>
int launch_decode_persistent(const AttnParams& p, cudaStream_t stream) {
  const size_t pipe = (size_t)4 * 3 * 2 * 16 * D * 2;
  const size_t merge = (size_t)(4 * 8 * D + 64) * 4;
  const size_t smem = pipe + merge;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    PG_CUDA(cudaGetDevice(&dev));
    PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    PG_CUDA(cudaFuncSetAttribute(decode_attn_persistent_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int units = p.num_seqs * p.hkv * p.splits;
  const int slots = sms * (D <= 128 ? 2 : 1);
  PG_CUDA(launch_pdl(decode_attn_persistent_kernel<D>, dim3(units < slots ? units : slots), dim3(128), smem, stream, p));
  PG_LAUNCH_CHECK();
  if (p.splits > 1) {
    PG_CUDA(launch_pdl(decode_merge_kernel<D>, dim3((p.num_seqs * p.hq + 3) / 4), dim3(128), (size_t)(0), stream, p));
    PG_LAUNCH_CHECK();
  }
  return PG_OK;
}

template <int D>
int launch_decode(const AttnParams& p, cudaStream_t stream) {
  if (g_decode_persistent < 0) {
    const char* e = getenv("PEGAINFER_ATTN_PERSISTENT");
    g_decode_persistent = (e && e[0] == '0') ? 0 : 1;
  }
  if (g_decode_persistent) return launch_decode_persistent<D>(p, stream);
  if (g_decode_stages == 2) return launch_decode_s<D, 2>(p, stream);
  return launch_decode_s<D, 3>(p, stream);
}

int g_prefill_ctas = 0;  // PEGAINFER_PREFILL_CTAS=2|3: register budget of the prefill kernel (CTAs per SM)

template <int D, int MINB>
int launch_prefill_b(const AttnParams& p, int q_tiles, int window, cudaStream_t stream) {
  const size_t smem = (size_t)2 * 2 * 64 * D * 2;
  static bool set = false;
  if (!set) {
    PG_CUDA(cudaFuncSetAttribute(prefill_attn_kernel<D, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  dim3 grid(q_tiles, p.hq);
  PG_CUDA(launch_pdl(prefill_attn_kernel<D, MINB>, dim3(grid), dim3(128), (size_t)(smem), stream, p, window));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

template <int D>
int launch_prefill(const AttnParams& p, int q_tiles, int window, cudaStream_t stream) {
  if (g_prefill_ctas == 0) {
    const char* e = getenv("PEGAINFER_PREFILL_CTAS");
    g_prefill_ctas = (e && e[0] == '3') ? 3 : 2;
  }
  if constexpr (D <= 128) {
    if (g_prefill_ctas == 3) return launch_prefill_b<D, 3>(p, q_tiles, window, stream);
  }
  return launch_prefill_b<D, (D <= 128 ? 2 : 1)>(p, q_tiles, window, stream);
}

}  // namespace

extern "C" void pg_attn_set_decode_stages(int stages) { g_decode_stages = stages == 2 ? 2 : 3; }

// Number of KV splits per (sequence, kv head): fill the resident CTA slots
// (`per_sm` CTAs per SM) with as little wave-quantisation loss as possible, keeping at
// least four 16-token tiles per split.
extern "C" int pg_decode_splits(int num_seqs, int hkv, int max_kv_len, int sms) {
  const int ctas = num_seqs * hkv;
  const int per_sm = g_decode_stages == 2 ? 3 : 2;
  const int slots = sms * per_sm;
  int max_by_len = (max_kv_len + 63) / 64;
  if (max_by_len < 1) max_by_len = 1;
  if (max_by_len > 32) max_by_len = 32;
  int best = 1;
  double best_score = -1.0;
  for (int s = 1; s <= max_by_len; ++s) {
    const long long total = (long long)ctas * s;
    const long long waves = (total + slots - 1) / slots;
    double eff = (double)total / (double)(waves * slots);
    eff -= 0.01 * (s - 1);  // each extra split costs merge traffic and a shorter main loop
    if (eff > best_score + 1e-9) {
      best_score = eff;
      best = s;
    }
  }
  return best;
}

// mode 0: decode (one query row per sequence), mode 1: prefill / mixed.
extern "C" int pg_paged_attention(const void* q, const void* kv, void* out, const void* q_indptr, const void* kv_lens, const void* table,
                                  int table_stride, int num_seqs, int hq, int hkv, int dim, int page_size, long long num_pages, float scale,
                                  int mode, int splits, void* part_o, void* part_lse, int q_tiles, int window, void* status,
                                  cudaStream_t stream) {
  PG_REQUIRE(dim == 64 || dim == 128 || dim == 256, "paged_attention: head_dim %d not supported (64, 128, 256)", dim);
  PG_REQUIRE(hq % hkv == 0 && hq / hkv <= 8, "paged_attention: GQA group %d/%d not supported (<= 8)", hq, hkv);
  PG_REQUIRE(page_size == 16 || page_size == 32 || page_size == 64, "paged_attention: page size %d not supported", page_size);
  if (num_seqs == 0) return PG_OK;
  AttnParams p;
  p.q = (const bf16*)q;
  p.kv = (const bf16*)kv;
  p.out = (bf16*)out;
  p.q_indptr = (const int*)q_indptr;
  p.kv_lens = (const int*)kv_lens;
  p.table = (const int*)table;
  p.table_stride = table_stride;
  p.num_seqs = num_seqs;
  p.hq = hq;
  p.hkv = hkv;
  p.page_size = page_size;
  p.scale_log2 = scale * LOG2E;
  p.splits = splits < 1 ? 1 : splits;
  p.part_o = (float*)part_o;
  p.part_lse = (float*)part_lse;
  p.num_pages = num_pages;
  p.status = (uint32_t*)status;
  p.window = mode == 0 ? window : 0;
  if (mode == 0) {
    PG_REQUIRE(p.splits == 1 || (part_o && part_lse), "paged_attention: split-KV decode needs partial buffers");
    if (dim == 64) return launch_decode<64>(p, stream);
    if (dim == 128) return launch_decode<128>(p, stream);
    return launch_decode<256>(p, stream);
  }
  if (q_tiles == 0) return PG_OK;
  if (dim == 64) return launch_prefill<64>(p, q_tiles, window, stream);
  if (dim == 128) return launch_prefill<128>(p, q_tiles, window, stream);
  return launch_prefill<256>(p, q_tiles, window, stream);
}
