// Gated DeltaNet prefill as a chunk-wise scan on the tensor cores.
//
// The gated delta rule  S <- a_t S;  d_t = b_t (v_t - S^T k_t);  S <- S + k_t d_t^T;  o_t = S^T q_t
// (S is the [Dk, Dv] state of one value head, a_t = exp(g_t) the decay, b_t = beta_t) is
// evaluated 64 tokens at a time.  With G_i the running sum of g inside the chunk and S0 the
// state at its start, the 64 corrections D = [d_0 .. d_63]^T solve a unit lower-triangular
// system
//     (I + A) D = beta .* (V - diag(exp G) K S0),   A_jl = beta_j exp(G_j - G_l) (k_j . k_l), l < j,
// so with T = (I + A)^-1:   D = T (beta V) - [T (beta exp(G) K)] S0 = U - W S0,
//     O  = diag(exp G) Q S0 + P D,           P_ij = exp(G_i - G_j) (q_i . k_j), j <= i,
//     S1 = exp(G_63) S0 + (exp(G_63 - G) K)^T D.
// Every product is a bf16 mma.sync with f32 accumulation; the state itself stays in f32
// registers (as the accumulator of the last product) for the whole sequence and is rounded to
// bf16 only as an operand.  All decay factors that appear are exp of a non-positive number.
// T comes from forward substitution in f32 (64 columns x 4 lanes, fully unrolled).  The raw
// rows of the next chunk are copied into a staging buffer by cp.async while the current
// chunk is processed.
//
// CTA = (sequence, value head, half of the Dv columns); 8 warps.  Takes the place of the
// reference's chunk-wise Triton pipeline (pegainfer-kernels/tools/triton/
// gated_delta_rule_chunkwise_kernels.py:28-708, chunk 64); the oracle is the token-by-token
// recurrence of gdn.cu.
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int C = 64;     // tokens per chunk
constexpr int DK = 128;   // key width
constexpr int DVC = 64;   // value columns per CTA
constexpr int LDK = DK + 8;   // padded row strides (bf16 elements): 16-byte shift per row, conflict-free ldmatrix
constexpr int LDV = DVC + 8;
constexpr int LDA = C + 1;    // f32 A matrix

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A fragment (16 x 16) of a row-major [m][k] matrix.
__device__ __forceinline__ void frag_a(const bf16* s, int ld, int m0, int k0, int lane, uint32_t* a) {
  const int row = m0 + (lane & 7) + ((lane >> 3) & 1) * 8, col = k0 + (lane >> 4) * 8;
  ldsm_x4(smem_u32(s + row * ld + col), a[0], a[1], a[2], a[3]);
}
// A fragment (16 x 16) of A[m][k] stored as [k][m].
__device__ __forceinline__ void frag_a_t(const bf16* s, int ld, int m0, int k0, int lane, uint32_t* a) {
  const int row = k0 + (lane & 7) + (lane >> 4) * 8, col = m0 + ((lane >> 3) & 1) * 8;
  ldsm_x4_t(smem_u32(s + row * ld + col), a[0], a[1], a[2], a[3]);
}
// B fragments of two 8-wide n-tiles (n0, n0 + 8) over 16 k, B[k][n] stored as [n][k].
__device__ __forceinline__ void frag_b_nk(const bf16* s, int ld, int n0, int k0, int lane, uint32_t* b) {
  const int j = lane >> 3, r = lane & 7;
  const int row = n0 + (j >> 1) * 8 + r, col = k0 + (j & 1) * 8;
  ldsm_x4(smem_u32(s + row * ld + col), b[0], b[1], b[2], b[3]);
}
// Same, B[k][n] stored as [k][n].
__device__ __forceinline__ void frag_b_kn(const bf16* s, int ld, int k0, int n0, int lane, uint32_t* b) {
  const int j = lane >> 3, r = lane & 7;
  const int row = k0 + (j & 1) * 8 + r, col = n0 + (j >> 1) * 8;
  ldsm_x4_t(smem_u32(s + row * ld + col), b[0], b[1], b[2], b[3]);
}

struct ChunkSmem {
  bf16 k[C * LDK];    // normalised keys
  bf16 q[C * LDK];    // normalised, scaled queries
  bf16 kg[C * LDK];   // beta_i exp(G_i) k_i
  bf16 kd[C * LDK];   // exp(G_last - G_i) k_i
  bf16 w[C * LDK];    // W = T (beta exp(G) K)
  bf16 vb[C * LDV];   // beta_i v_i
  bf16 t[C * LDV];    // T = (I + A)^-1
  bf16 p[C * LDV];    // masked, decayed Q K^T
  bf16 d[C * LDV];    // D = U - W S0
  bf16 s[DK * LDV];   // bf16 copy of the state, [dk][dv]
  bf16 raw_k[C * LDK];  // next chunk's raw k, q, v rows (cp.async staging, filled while this chunk is processed)
  bf16 raw_q[C * LDK];
  bf16 raw_v[C * LDV];
  float a[C * LDA];   // A (strictly lower part is used)
  float gsum[C];      // G_i
  float beta[C];
};

__global__ void __launch_bounds__(256, 1)
gdn_chunk_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, long long ld_qk, const bf16* __restrict__ v, long long ld_v,
                 const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state, bf16* __restrict__ out,
                 const int* __restrict__ q_indptr, const int* __restrict__ slots, int hk, int hv, int dv, int min_len) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  ChunkSmem& sm = *reinterpret_cast<ChunkSmem*>(smem_raw);
  const int splits = dv / DVC;
  const int h = blockIdx.x / splits, dv0 = (blockIdx.x % splits) * DVC, b = blockIdx.y;
  const int slot = slots[b];
  const int q0 = q_indptr[b], q1 = q_indptr[b + 1];
  if (q1 - q0 < min_len || q1 == q0 || slot < 0) return;
  const int kh = h / (hv / hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, t4 = lane & 3;
  const int wm = warp & 3, wn = warp >> 2;  // token tile (16 rows) and column half of the 64-row products
  const float q_scale = rsqrtf((float)DK);

  // state: warp w owns rows [16w, 16w + 16) of S[dk][dv0 .. dv0 + 64) as mma accumulators
  float* S = state + (((long long)slot * hv + h) * DK) * dv + dv0;
  float sacc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int col = n * 8 + 2 * t4;
    const float2 lo = *reinterpret_cast<const float2*>(S + (long long)(warp * 16 + gq) * dv + col);
    const float2 hi = *reinterpret_cast<const float2*>(S + (long long)(warp * 16 + gq + 8) * dv + col);
    sacc[n][0] = lo.x;
    sacc[n][1] = lo.y;
    sacc[n][2] = hi.x;
    sacc[n][3] = hi.y;
    *reinterpret_cast<uint32_t*>(&sm.s[(warp * 16 + gq) * LDV + col]) = pack2(lo.x, lo.y);
    *reinterpret_cast<uint32_t*>(&sm.s[(warp * 16 + gq + 8) * LDV + col]) = pack2(hi.x, hi.y);
  }

  // Raw rows of a chunk go to shared memory by cp.async (rows past the sequence end are
  // zero-filled); the copy of chunk c + 1 is started once chunk c has been read out of the
  // staging buffers and lands while chunk c is processed.
  auto stage_chunk = [&](int t0) {
    const int nt = min(C, q1 - t0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = tid + 256 * i, r = c >> 4, ch = c & 15;  // 64 rows x 16 chunks of 8 elements
      const bool ok = r < nt;
      const long long src_row = (long long)(t0 + (ok ? r : 0)) * ld_qk + (long long)kh * DK + ch * 8;
      cp_async16(&sm.raw_k[r * LDK + ch * 8], k + src_row, ok);
      cp_async16(&sm.raw_q[r * LDK + ch * 8], q + src_row, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + 256 * i, r = c >> 3, ch = c & 7;  // 64 rows x 8 chunks
      const bool ok = r < nt;
      cp_async16(&sm.raw_v[r * LDV + ch * 8], v + (long long)(t0 + (ok ? r : 0)) * ld_v + (long long)h * dv + dv0 + ch * 8, ok);
    }
    cp_async_commit();
  };
  stage_chunk(q0);

  for (int t0 = q0; t0 < q1; t0 += C) {
    const int nt = min(C, q1 - t0);
    // ---- phase A: normalise the staged rows, decay sums ---------------------------------
    // thread = (row = tid / 4, quarter = tid % 4): 32 elements of q and k of one token
    const int row = tid >> 2, qt = tid & 3;
    float kf[32], qf[32];
    float g_raw = 0.f, b_raw = 0.f;
    if (warp < 2) {
      const int r = warp * 32 + lane;
      if (r < nt) {
        g_raw = g[(long long)(t0 + r) * hv + h];
        b_raw = beta[(long long)(t0 + r) * hv + h];
      }
    }
    cp_async_wait_all();
    __syncthreads();
    {
      float ks = 0.f, qs = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bf16x8 kk = *reinterpret_cast<const bf16x8*>(&sm.raw_k[row * LDK + qt * 32 + i * 8]);
        const bf16x8 qq = *reinterpret_cast<const bf16x8*>(&sm.raw_q[row * LDK + qt * 32 + i * 8]);
        float kt[8], qtmp[8];
        unpack8(kk, kt);
        unpack8(qq, qtmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          kf[i * 8 + e] = kt[e];
          qf[i * 8 + e] = qtmp[e];
          ks += kf[i * 8 + e] * kf[i * 8 + e];
          qs += qf[i * 8 + e] * qf[i * 8 + e];
        }
      }
      ks += __shfl_xor_sync(0xffffffffu, ks, 1);
      ks += __shfl_xor_sync(0xffffffffu, ks, 2);
      qs += __shfl_xor_sync(0xffffffffu, qs, 1);
      qs += __shfl_xor_sync(0xffffffffu, qs, 2);
      const float kn = rsqrtf(ks + 1e-6f), qn = rsqrtf(qs + 1e-6f) * q_scale;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        kf[i] *= kn;
        qf[i] *= qn;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        *reinterpret_cast<uint32_t*>(&sm.k[row * LDK + qt * 32 + 2 * i]) = pack2(kf[2 * i], kf[2 * i + 1]);
        *reinterpret_cast<uint32_t*>(&sm.q[row * LDK + qt * 32 + 2 * i]) = pack2(qf[2 * i], qf[2 * i + 1]);
      }
    }
    if (warp < 2) {
      // inclusive scan of g over the 64 rows (two warps, the second adds the first's total)
      const int r = warp * 32 + lane;
      float x = g_raw;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      sm.gsum[r] = x;  // warp 1 holds partial sums until the fix-up below
      sm.beta[r] = b_raw;
    }
    __syncthreads();
    if (warp == 1) sm.gsum[32 + lane] += sm.gsum[31];
    __syncthreads();
    {
      const float gi = sm.gsum[row], bi = sm.beta[row], glast = sm.gsum[C - 1];
      const float fg = bi * __expf(gi), fd = __expf(glast - gi);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        *reinterpret_cast<uint32_t*>(&sm.kg[row * LDK + qt * 32 + 2 * i]) = pack2(kf[2 * i] * fg, kf[2 * i + 1] * fg);
        *reinterpret_cast<uint32_t*>(&sm.kd[row * LDK + qt * 32 + 2 * i]) = pack2(kf[2 * i] * fd, kf[2 * i + 1] * fd);
      }
      // beta * V: 16 columns of this token per thread
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float vt[8];
        const bf16x8 vv = *reinterpret_cast<const bf16x8*>(&sm.raw_v[row * LDV + qt * 16 + i * 8]);
        unpack8(vv, vt);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          *reinterpret_cast<uint32_t*>(&sm.vb[row * LDV + qt * 16 + i * 8 + 2 * e]) = pack2(vt[2 * e] * bi, vt[2 * e + 1] * bi);
      }
    }
    __syncthreads();
    if (t0 + C < q1) stage_chunk(t0 + C);  // every thread has read this chunk out of the staging buffers

    // ---- phase B: K K^T and Q K^T (64 x 64 each), warp = 16 rows x 32 columns ----------
    {
      float kk[4][4], qk[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) kk[n][e] = qk[n][e] = 0.f;
      // rows of the warp's tile are >= its columns only if 16 wm + 15 >= 32 wn: tiles above the diagonal stay zero
      if (wm * 16 + 15 >= wn * 32) {
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
          uint32_t ak[4], aq[4], b0[4], b1[4];
          frag_a(sm.k, LDK, wm * 16, ks * 16, lane, ak);
          frag_a(sm.q, LDK, wm * 16, ks * 16, lane, aq);
          frag_b_nk(sm.k, LDK, wn * 32, ks * 16, lane, b0);
          frag_b_nk(sm.k, LDK, wn * 32 + 16, ks * 16, lane, b1);
          mma16816(kk[0], ak, b0[0], b0[1]);
          mma16816(kk[1], ak, b0[2], b0[3]);
          mma16816(kk[2], ak, b1[0], b1[1]);
          mma16816(kk[3], ak, b1[2], b1[3]);
          mma16816(qk[0], aq, b0[0], b0[1]);
          mma16816(qk[1], aq, b0[2], b0[3]);
          mma16816(qk[2], aq, b1[0], b1[1]);
          mma16816(qk[3], aq, b1[2], b1[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = wm * 16 + gq + (e >> 1) * 8, j = wn * 32 + n * 8 + 2 * t4 + (e & 1);
          const float dec = j <= i ? __expf(sm.gsum[i] - sm.gsum[j]) : 0.f;
          sm.a[i * LDA + j] = j < i ? sm.beta[i] * dec * kk[n][e] : 0.f;
          qk[n][e] *= dec;
        }
        const int j0 = wn * 32 + n * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(&sm.p[(wm * 16 + gq) * LDV + j0]) = pack2(qk[n][0], qk[n][1]);
        *reinterpret_cast<uint32_t*>(&sm.p[(wm * 16 + gq + 8) * LDV + j0]) = pack2(qk[n][2], qk[n][3]);
      }
    }
    __syncthreads();

    // ---- phase C: T = (I + A)^-1 by forward substitution --------------------------------
    {
      const int c = tid >> 2, part = tid & 3;  // column of T, and which rows l = 4 j + part this lane keeps
      float tcol[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) tcol[j] = 0.f;
#pragma unroll
      for (int i = 0; i < C; ++i) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < (i + 3) / 4; ++j) {
          const int l = 4 * j + part;
          if (l < i) s += sm.a[i * LDA + l] * tcol[j];
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        const float val = (i == c ? 1.f : 0.f) - s;
        if (part == (i & 3)) tcol[i >> 2] = val;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.t[(4 * j + part) * LDV + c] = __float2bfloat16(tcol[j]);
    }
    __syncthreads();

    // ---- phase D: U = T (beta V) in registers, W = T (beta exp(G) K) to shared ----------
    float u[4][4];
    {
      float wacc[8][4];
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) u[n][e] = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) wacc[n][e] = 0.f;
      // T is lower triangular: k-steps beyond the tile's rows contribute nothing
      for (int ks = 0; ks <= wm; ++ks) {
        uint32_t a[4], bb[4];
        frag_a(sm.t, LDV, wm * 16, ks * 16, lane, a);
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {
          frag_b_kn(sm.vb, LDV, ks * 16, wn * 32 + n2 * 16, lane, bb);
          mma16816(u[2 * n2], a, bb[0], bb[1]);
          mma16816(u[2 * n2 + 1], a, bb[2], bb[3]);
        }
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          frag_b_kn(sm.kg, LDK, ks * 16, wn * 64 + n2 * 16, lane, bb);
          mma16816(wacc[2 * n2], a, bb[0], bb[1]);
          mma16816(wacc[2 * n2 + 1], a, bb[2], bb[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = wn * 64 + n * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(&sm.w[(wm * 16 + gq) * LDK + col]) = pack2(wacc[n][0], wacc[n][1]);
        *reinterpret_cast<uint32_t*>(&sm.w[(wm * 16 + gq + 8) * LDK + col]) = pack2(wacc[n][2], wacc[n][3]);
      }
    }
    __syncthreads();

    // ---- phase E: D = U - W S0, and the state part of the output exp(G) Q S0 --------------
    float o[4][4];
    {
      float ws[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) ws[n][e] = o[n][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
        uint32_t aw[4], aq[4], bb[4];
        frag_a(sm.w, LDK, wm * 16, ks * 16, lane, aw);
        frag_a(sm.q, LDK, wm * 16, ks * 16, lane, aq);
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {
          frag_b_kn(sm.s, LDV, ks * 16, wn * 32 + n2 * 16, lane, bb);
          mma16816(ws[2 * n2], aw, bb[0], bb[1]);
          mma16816(ws[2 * n2 + 1], aw, bb[2], bb[3]);
          mma16816(o[2 * n2], aq, bb[0], bb[1]);
          mma16816(o[2 * n2 + 1], aq, bb[2], bb[3]);
        }
      }
      const float e_lo = __expf(sm.gsum[wm * 16 + gq]), e_hi = __expf(sm.gsum[wm * 16 + gq + 8]);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = wn * 32 + n * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(&sm.d[(wm * 16 + gq) * LDV + col]) = pack2(u[n][0] - ws[n][0], u[n][1] - ws[n][1]);
        *reinterpret_cast<uint32_t*>(&sm.d[(wm * 16 + gq + 8) * LDV + col]) = pack2(u[n][2] - ws[n][2], u[n][3] - ws[n][3]);
        o[n][0] *= e_lo;
        o[n][1] *= e_lo;
        o[n][2] *= e_hi;
        o[n][3] *= e_hi;
      }
    }
    __syncthreads();

    // ---- phase F: O += P D; S <- exp(G_last) S + (exp(G_last - G) K)^T D ------------------
    {
      for (int ks = 0; ks <= wm; ++ks) {  // P is lower triangular
        uint32_t a[4], bb[4];
        frag_a(sm.p, LDV, wm * 16, ks * 16, lane, a);
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {
          frag_b_kn(sm.d, LDV, ks * 16, wn * 32 + n2 * 16, lane, bb);
          mma16816(o[2 * n2], a, bb[0], bb[1]);
          mma16816(o[2 * n2 + 1], a, bb[2], bb[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = dv0 + wn * 32 + n * 8 + 2 * t4;
        const int r_lo = wm * 16 + gq, r_hi = r_lo + 8;
        if (r_lo < nt) *reinterpret_cast<uint32_t*>(out + ((long long)(t0 + r_lo) * hv + h) * dv + col) = pack2(o[n][0], o[n][1]);
        if (r_hi < nt) *reinterpret_cast<uint32_t*>(out + ((long long)(t0 + r_hi) * hv + h) * dv + col) = pack2(o[n][2], o[n][3]);
      }
      const float glast = __expf(sm.gsum[C - 1]);
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[n][e] *= glast;
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {
        uint32_t a[4], bb[4];
        frag_a_t(sm.kd, LDK, warp * 16, ks * 16, lane, a);
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          frag_b_kn(sm.d, LDV, ks * 16, n2 * 16, lane, bb);
          mma16816(sacc[2 * n2], a, bb[0], bb[1]);
          mma16816(sacc[2 * n2 + 1], a, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();  // every warp has read the old bf16 state (phase E) and D
    if (t0 + C < q1) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = n * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(&sm.s[(warp * 16 + gq) * LDV + col]) = pack2(sacc[n][0], sacc[n][1]);
        *reinterpret_cast<uint32_t*>(&sm.s[(warp * 16 + gq + 8) * LDV + col]) = pack2(sacc[n][2], sacc[n][3]);
      }
    }
    // the next chunk's first barrier orders these writes before phase E reads them
  }
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int col = n * 8 + 2 * t4;
    *reinterpret_cast<float2*>(S + (long long)(warp * 16 + gq) * dv + col) = make_float2(sacc[n][0], sacc[n][1]);
    *reinterpret_cast<float2*>(S + (long long)(warp * 16 + gq + 8) * dv + col) = make_float2(sacc[n][2], sacc[n][3]);
  }
}

}  // namespace

// Chunk-wise gated delta rule for every sequence of at least `min_len` tokens (shorter ones,
// decode rows in particular, are left to pg_gdn_recurrent).  dk must be 128, dv a multiple of 64.
extern "C" int pg_gdn_chunked(const void* q, const void* k, long long ld_qk, const void* v, long long ld_v, const void* g, const void* beta,
                              void* state, void* out, const void* q_indptr, const void* slots, int num_seqs, int hk, int hv, int dk, int dv,
                              int min_len, cudaStream_t stream) {
  PG_REQUIRE(dk == DK && dv % DVC == 0 && hv % hk == 0, "gdn_chunked: dk=%d must be 128, dv=%d a multiple of 64", dk, dv);
  PG_REQUIRE(ld_qk % 8 == 0 && ld_v % 8 == 0, "gdn_chunked: row strides must be multiples of 8 elements");
  PG_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && (((uintptr_t)state | (uintptr_t)out) & 7) == 0,
             "gdn_chunked: q, k, v must be 16-byte aligned, state and out 8-byte aligned");
  if (num_seqs == 0) return PG_OK;
  static bool set = false;
  if (!set) {
    PG_CUDA(cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ChunkSmem)));
    set = true;
  }
  dim3 grid(hv * (dv / DVC), num_seqs);
  gdn_chunk_kernel<<<grid, 256, sizeof(ChunkSmem), stream>>>((const bf16*)q, (const bf16*)k, ld_qk, (const bf16*)v, ld_v, (const float*)g,
                                                              (const float*)beta, (float*)state, (bf16*)out, (const int*)q_indptr,
                                                              (const int*)slots, hk, hv, dv, min_len);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
