// Multi-head latent attention kernels (DeepSeek-V2-Lite / Kimi-K2 shapes).
//
//  * mla_append: RMSNorm of the compressed KV row, RoPE of the shared rope key
//    (interleaved-pair input -> half-split output), append [ckv | k_pe] to the paged
//    latent cache [pages, page_size, kv_lora + rope].
//  * mla_q_prep: RoPE on the query rope tail and a head-major copy of q_nope, so the
//    absorb step (q_nope * W_UK per head) can run on the grouped tcgen05 GEMM.
//  * mla_attn: absorbed attention over the latent cache.  All heads share one KV row per
//    token, so a CTA takes 16 heads of one query token as the 16 MMA rows and streams
//    32-token latent tiles (cp.async, double buffered).  The 576-wide score contraction
//    is split over the four warps (9 k-steps each) and summed through shared memory;
//    each warp then owns 128 of the 512 value dims for P*V.  Split-KV + merge for decode.
//  * permute_021: [A, B, D] -> [B, A, D] row permutation (head-major <-> token-major).
//
// Functional parity with pegainfer-kernels/csrc/kimi_k2/kimi_mla.cu:83-885 (split/norm,
// rope, paged append, absorbed batch decode), csrc/deepseek_v2_lite/dsv2_lite_attention.cu
// and csrc/k3/k3_mla_paged_attn.cu (block-table walk, zero output for empty rows).
#include <float.h>

#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
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

// one warp per token
__global__ void __launch_bounds__(128) mla_append_kernel(const bf16* __restrict__ kv_a, long long ld, const bf16* __restrict__ norm_w,
                                                          const bf16* __restrict__ cos, const bf16* __restrict__ sin, const int* __restrict__ positions,
                                                          const int* __restrict__ slots, bf16* __restrict__ latent, int tokens, int c, int rope,
                                                          int max_pos, long long num_slots, float eps, uint32_t* status) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const long long slot = slots[t];
  if (slot < 0 || slot >= num_slots) {
    if (lane == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (6u << 8));
    return;
  }
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    if (lane == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (7u << 8));
    pos = pos < 0 ? 0 : max_pos - 1;
  }
  const bf16* src = kv_a + t * ld;
  bf16* dst = latent + slot * (c + rope);
  float ss = 0.f;
  for (int i = lane; i < c; i += 32) {
    const float v = __bfloat162float(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)c + eps);
  for (int i = lane; i < c; i += 32) dst[i] = __float2bfloat16(__bfloat162float(src[i]) * inv * __bfloat162float(norm_w[i]));
  const int half = rope / 2;
  for (int i = lane; i < half; i += 32) {
    const float x1 = __bfloat162float(src[c + 2 * i]), x2 = __bfloat162float(src[c + 2 * i + 1]);
    const float cs = __bfloat162float(cos[(long long)pos * half + i]), sn = __bfloat162float(sin[(long long)pos * half + i]);
    dst[c + i] = __float2bfloat16(x1 * cs - x2 * sn);
    dst[c + half + i] = __float2bfloat16(x2 * cs + x1 * sn);
  }
}

// one warp per (token, head): q [T, H, nope + rope] -> q_nope_hm [H, T, nope], q_pe [T, H, rope] (rotated)
__global__ void __launch_bounds__(128) mla_q_prep_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cos, const bf16* __restrict__ sin,
                                                          const int* __restrict__ positions, bf16* __restrict__ q_nope_hm, bf16* __restrict__ q_pe,
                                                          int tokens, int heads, int nope, int rope, int max_pos) {
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= (long long)tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  const bf16* src = q + unit * (nope + rope);
  bf16* dn = q_nope_hm + ((long long)h * tokens + t) * nope;
  for (int i = lane; i < nope / 8; i += 32) reinterpret_cast<uint4*>(dn)[i] = reinterpret_cast<const uint4*>(src)[i];
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const int half = rope / 2;
  bf16* dp = q_pe + unit * rope;
  for (int i = lane; i < half; i += 32) {
    const float x1 = __bfloat162float(src[nope + 2 * i]), x2 = __bfloat162float(src[nope + 2 * i + 1]);
    const float cs = __bfloat162float(cos[(long long)pos * half + i]), sn = __bfloat162float(sin[(long long)pos * half + i]);
    dp[i] = __float2bfloat16(x1 * cs - x2 * sn);
    dp[half + i] = __float2bfloat16(x2 * cs + x1 * sn);
  }
}

__global__ void permute_021_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int A, int B, int D) {
  const long long row = blockIdx.x;  // output row index b * A + a
  const int b = (int)(row / A), a = (int)(row % A);
  const uint4* src = reinterpret_cast<const uint4*>(in + ((long long)a * B + b) * D);
  uint4* dst = reinterpret_cast<uint4*>(out + row * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

struct MlaParams {
  const bf16* q_abs;   // [H, T, C] head-major
  const bf16* q_pe;    // [T, H, R]
  const bf16* latent;  // [pages, ps, C + R]
  bf16* out;           // [H, T, C] head-major
  const int* q_indptr;
  const int* kv_lens;
  const int* table;
  int table_stride, num_seqs, tokens, heads, page_size, splits;
  float scale_log2;
  float* part_o;    // [units, splits, C]
  float* part_lse;  // [units, splits, 16]
  const int* unit_seq;  // [T] sequence of each token row
};

// CTA = (token row t, head group of 16, split).  C = 512, R = 64 fixed by the template.
template <int C, int R>
__global__ void __launch_bounds__(128) mla_attn_kernel(const MlaParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int W = C + R;          // 576
  constexpr int TILE = 32;
  constexpr int CHUNKS = W / 8;     // 72 sixteen-byte chunks per row
  constexpr int KS_PER_WARP = (W / 16) / 4;  // 9
  constexpr int VD = C / 4;         // 128 value dims per warp
  constexpr int NT = VD / 8;        // 16
  bf16* tile_sm = reinterpret_cast<bf16*>(smem_raw);                           // [2][TILE][W]
  float* s_part = reinterpret_cast<float*>(smem_raw + 2 * TILE * W * 2);     // [4 warps][16][TILE]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int groups = p.heads / 16;
  const int split = blockIdx.x % p.splits;
  const int hg = (blockIdx.x / p.splits) % groups;
  const int t = blockIdx.x / (p.splits * groups);
  const int b = p.unit_seq[t];
  const int q0 = p.q_indptr[b], q1 = p.q_indptr[b + 1];
  const int kv_len = p.kv_lens[b];
  const int pos = kv_len - (q1 - q0) + (t - q0);  // position of this query token
  const int kv_end = kv_len == 0 ? 0 : pos + 1;   // causal
  const int* table_row = p.table + (long long)b * p.table_stride;
  const int n_tiles = (kv_end + TILE - 1) / TILE;
  const int tps = (n_tiles + p.splits - 1) / p.splits;
  const int t_begin = split * tps, t_end = min(n_tiles, t_begin + tps);

  auto swz = [](int r, int ch) { return r * W + ((ch ^ (r & 7)) << 3); };

  // Q fragments for this warp's K slice: dims [warp*144, warp*144 + 144) of [q_abs | q_pe]
  uint32_t qf[KS_PER_WARP][4];
#pragma unroll
  for (int ks = 0; ks < KS_PER_WARP; ++ks) {
    const int d0 = (warp * KS_PER_WARP + ks) * 16;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int head = hg * 16 + g + rr * 8;
        const int d = d0 + half * 8 + 2 * t4;
        uint32_t v;
        if (d < C)
          v = *reinterpret_cast<const uint32_t*>(p.q_abs + ((long long)head * p.tokens + t) * C + d);
        else
          v = *reinterpret_cast<const uint32_t*>(p.q_pe + ((long long)t * p.heads + head) * R + (d - C));
        qf[ks][half * 2 + rr] = v;
      }
    }
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};

  // A 32-token tile starts at a multiple of 32 and pages hold 16, 32 or 64 tokens: at most two
  // page-table entries per tile, read once; a thread's 18 chunks follow by stepping (row, chunk)
  // instead of dividing by 72 and by the page size for every 16 bytes.
  const int ps_shift = __ffs(p.page_size) - 1;
  const int c0_r = threadIdx.x / CHUNKS, c0_ch = threadIdx.x % CHUNKS;
  auto issue = [&](int tile, int stage) {
    bf16* dst = tile_sm + stage * TILE * W;
    if (tile < t_end) {
      const int tok_base = tile * TILE;
      const int pf = tok_base >> ps_shift;
      const int pg0 = table_row[min(pf, p.table_stride - 1)];
      const int pg1 = (1 << ps_shift) < TILE ? table_row[min(pf + 1, p.table_stride - 1)] : pg0;
      int r = c0_r, ch = c0_ch;
#pragma unroll
      for (int i = 0; i < TILE * CHUNKS / 128; ++i) {
        const bool valid = tok_base + r < kv_end;
        const int rr = valid ? r : 0;
        const int page = (rr >> ps_shift) ? pg1 : pg0;
        const bf16* src = p.latent + ((long long)page * p.page_size + ((tok_base + rr) & (p.page_size - 1))) * W + ch * 8;
        cp_async16(dst + swz(r, ch), src, valid);
        ch += 128 % CHUNKS;
        r += 128 / CHUNKS;
        if (ch >= CHUNKS) {
          ch -= CHUNKS;
          ++r;
        }
      }
    }
    cp_async_commit();
  };

  issue(t_begin, 0);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int stage = (tile - t_begin) & 1;
    issue(tile + 1, stage ^ 1);
    cp_async_wait<1>();
    __syncthreads();
    const bf16* ts = tile_sm + stage * TILE * W;
    // partial scores over this warp's 144 dims: [16 heads x 32 tokens]
    float s_acc[TILE / 8][4];
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n) s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS_PER_WARP; ++ks) {
      const int chb = (warp * KS_PER_WARP + ks) * 2;
#pragma unroll
      for (int n2 = 0; n2 < TILE / 16; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = n2 * 16 + (j >> 1) * 8 + r;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(ts + swz(row, chb + (j & 1))), b0, b1, b2, b3);
        mma16816(s_acc[2 * n2], qf[ks], b0, b1);
        mma16816(s_acc[2 * n2 + 1], qf[ks], b2, b3);
      }
    }
    float* mine = s_part + warp * 16 * TILE;
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n) {
      mine[g * TILE + n * 8 + 2 * t4] = s_acc[n][0];
      mine[g * TILE + n * 8 + 2 * t4 + 1] = s_acc[n][1];
      mine[(g + 8) * TILE + n * 8 + 2 * t4] = s_acc[n][2];
      mine[(g + 8) * TILE + n * 8 + 2 * t4 + 1] = s_acc[n][3];
    }
    __syncthreads();
    float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = g + (e >> 1) * 8, col = n * 8 + 2 * t4 + (e & 1);
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) s += s_part[(w * 16 + row) * TILE + col];
        const int tok = tile * TILE + col;
        s = tok < kv_end ? s * p.scale_log2 : NEG_BIG;
        s_acc[n][e] = s;
        mx[e >> 1] = fmaxf(mx[e >> 1], s);
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
    uint32_t pa[TILE / 16][4];
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[e] = s_acc[n][e] <= NEG_BIG ? 0.f : exp2f(s_acc[n][e] - m_run[e >> 1]);
        ps[e >> 1] += pv[e];
      }
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
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
    // P * V over this warp's 128 value dims
#pragma unroll
    for (int kk = 0; kk < TILE / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = kk * 16 + (j & 1) * 8 + r;
        const int ch = warp * (VD / 8) + n2 * 2 + (j >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(ts + swz(row, ch)), b0, b1, b2, b3);
        mma16816(o[2 * n2], pa[kk], b0, b1);
        mma16816(o[2 * n2 + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();  // tile and s_part are reused by the next iteration
  }
  cp_async_wait<0>();

  // every warp holds the same (m, l); it writes its own 128 value dims
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int head = hg * 16 + g + rr * 8;
    const float L = l_run[rr];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    if (p.splits == 1) {
      bf16* dst = p.out + ((long long)head * p.tokens + t) * C + warp * VD;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
    } else {
      const long long unit = ((long long)t * groups + hg) * 16 + g + rr * 8;  // (token, head) index
      float* dst = p.part_o + (unit * p.splits + split) * C + warp * VD;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        dst[n * 8 + 2 * t4] = o[n][rr * 2] * inv;
        dst[n * 8 + 2 * t4 + 1] = o[n][rr * 2 + 1] * inv;
      }
      if (warp == 0 && t4 == 0) p.part_lse[unit * p.splits + split] = L > 0.f ? m_run[rr] + log2f(L) : NEG_BIG;
    }
  }
}

template <int C>
__global__ void __launch_bounds__(128) mla_merge_kernel(const MlaParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;  // (token, head)
  if (unit >= (long long)p.tokens * p.heads) return;
  const int t = (int)(unit / p.heads), head = (int)(unit % p.heads);
  const float* lse = p.part_lse + unit * p.splits;
  float M = NEG_BIG;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, lse[s]);
  float acc[C / 32];
#pragma unroll
  for (int i = 0; i < C / 32; ++i) acc[i] = 0.f;
  float Wsum = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    if (lse[s] <= NEG_BIG) continue;
    const float f = exp2f(lse[s] - M);
    Wsum += f;
    const float* po = p.part_o + (unit * p.splits + s) * C;
#pragma unroll
    for (int i = 0; i < C / 32; ++i) acc[i] += f * po[lane + 32 * i];
  }
  bf16* dst = p.out + ((long long)head * p.tokens + t) * C;
#pragma unroll
  for (int i = 0; i < C / 32; ++i) dst[lane + 32 * i] = __float2bfloat16(Wsum > 0.f ? acc[i] / Wsum : 0.f);
}

}  // namespace

extern "C" int pg_mla_append(const void* kv_a, long long ld, const void* norm_w, const void* cos, const void* sin, const void* positions,
                             const void* slots, void* latent, int tokens, int c, int rope, int max_pos, long long num_slots, float eps,
                             void* status, cudaStream_t stream) {
  if (tokens == 0) return PG_OK;
  mla_append_kernel<<<(tokens + 3) / 4, 128, 0, stream>>>((const bf16*)kv_a, ld, (const bf16*)norm_w, (const bf16*)cos, (const bf16*)sin,
                                                         (const int*)positions, (const int*)slots, (bf16*)latent, tokens, c, rope, max_pos,
                                                         num_slots, eps, (uint32_t*)status);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_mla_q_prep(const void* q, const void* cos, const void* sin, const void* positions, void* q_nope_hm, void* q_pe, int tokens,
                             int heads, int nope, int rope, int max_pos, cudaStream_t stream) {
  PG_REQUIRE(nope % 8 == 0 && rope % 2 == 0, "mla_q_prep: nope %d / rope %d not supported", nope, rope);
  if (tokens == 0) return PG_OK;
  const long long units = (long long)tokens * heads;
  mla_q_prep_kernel<<<(unsigned)((units + 3) / 4), 128, 0, stream>>>((const bf16*)q, (const bf16*)cos, (const bf16*)sin, (const int*)positions,
                                                                    (bf16*)q_nope_hm, (bf16*)q_pe, tokens, heads, nope, rope, max_pos);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_permute_021(const void* in, void* out, int A, int B, int D, cudaStream_t stream) {
  PG_REQUIRE(D % 8 == 0, "permute: inner dim %d must be a multiple of 8", D);
  if ((long long)A * B == 0) return PG_OK;
  permute_021_kernel<<<(unsigned)((long long)A * B), 64, 0, stream>>>((const bf16*)in, (bf16*)out, A, B, D);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_mla_attention(const void* q_abs, const void* q_pe, const void* latent, void* out, const void* q_indptr, const void* kv_lens,
                                const void* table, int table_stride, const void* unit_seq, int num_seqs, int tokens, int heads, int c, int rope,
                                int page_size, float scale, int splits, void* part_o, void* part_lse, void* status, cudaStream_t stream) {
  PG_REQUIRE(c == 512 && rope == 64, "mla_attention: built for kv_lora 512 + rope 64 (got %d + %d)", c, rope);
  PG_REQUIRE(heads % 16 == 0, "mla_attention: heads %d must be a multiple of 16", heads);
  if (tokens == 0) return PG_OK;
  MlaParams p;
  p.q_abs = (const bf16*)q_abs;
  p.q_pe = (const bf16*)q_pe;
  p.latent = (const bf16*)latent;
  p.out = (bf16*)out;
  p.q_indptr = (const int*)q_indptr;
  p.kv_lens = (const int*)kv_lens;
  p.table = (const int*)table;
  p.table_stride = table_stride;
  p.num_seqs = num_seqs;
  p.tokens = tokens;
  p.heads = heads;
  p.page_size = page_size;
  p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * LOG2E;
  p.part_o = (float*)part_o;
  p.part_lse = (float*)part_lse;
  p.unit_seq = (const int*)unit_seq;
  PG_REQUIRE(p.splits == 1 || (part_o && part_lse), "mla_attention: split-KV needs partial buffers");
  const size_t smem = (size_t)2 * 32 * 576 * 2 + 4 * 16 * 32 * 4;
  static bool set = false;
  if (!set) {
    PG_CUDA(cudaFuncSetAttribute(mla_attn_kernel<512, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  const int grid = tokens * (heads / 16) * p.splits;
  mla_attn_kernel<512, 64><<<grid, 128, smem, stream>>>(p);
  PG_LAUNCH_CHECK();
  if (p.splits > 1) {
    mla_merge_kernel<512><<<(unsigned)(((long long)tokens * heads + 3) / 4), 128, 0, stream>>>(p);
    PG_LAUNCH_CHECK();
  }
  return PG_OK;
}
