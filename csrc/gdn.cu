// Gated DeltaNet kernels (Qwen3.5 linear-attention layers).
//
//  * gdn_conv1d: causal depthwise conv (kernel <= 4) + SiLU over ragged sequences with a
//    carried [C, K-1] input history per sequence slot (prefill and decode in one kernel).
//  * gdn_gates: g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b).
//  * gdn_recurrent: the gated delta rule.  The columns of the f32 state S[Dk, Dv] evolve
//    independently, so a CTA takes 32 columns of one (sequence, value head) and four lanes
//    of a warp share a column, each keeping a quarter of its Dk elements in registers:
//    S^T k, the rank-1 update and S^T q are register dot products plus two shuffles, and a
//    single long prompt already spreads over heads x Dv/32 CTAs.  A decode step is one pass
//    over the state (read + write: HBM bound); a prefill chunk walks its tokens in order
//    with the state resident in registers.
//
// Functional parity with pegainfer-kernels/csrc/qwen35/conv1d.cu:19-165,
// gated_delta_rule.cu:28-347 and the chunk-wise Triton prefill pipeline
// (tools/triton/gated_delta_rule_chunkwise_kernels.py), whose result equals this
// recurrence.
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace {

__global__ void gdn_conv1d_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w, bf16* __restrict__ state,
                                  bf16* __restrict__ out, long long ldo, const int* __restrict__ q_indptr, const int* __restrict__ slots,
                                  int channels, int K, long long state_slot_stride) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int q0 = q_indptr[b], q1 = q_indptr[b + 1];
  const int slot = slots[b];
  if (q1 == q0) return;
  if (slot < 0) {
    for (int t = q0; t < q1; ++t) out[t * ldo + c] = __float2bfloat16(0.f);
    return;
  }
  bf16* st = state + slot * state_slot_stride + (long long)c * (K - 1);
  float hist[3] = {0.f, 0.f, 0.f};  // oldest .. newest of the last K-1 inputs
  for (int i = 0; i < K - 1; ++i) hist[3 - (K - 1) + i] = __bfloat162float(st[i]);
  float wt[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < K; ++i) wt[4 - K + i] = __bfloat162float(w[(long long)c * K + i]);
  for (int t = q0; t < q1; ++t) {
    const float cur = __bfloat162float(x[t * ldx + c]);
    float pre = hist[0] * wt[0] + hist[1] * wt[1] + hist[2] * wt[2] + cur * wt[3];
    pre = bf16_round(pre);
    out[t * ldo + c] = __float2bfloat16(pre / (1.f + __expf(-pre)));
    hist[0] = hist[1];
    hist[1] = hist[2];
    hist[2] = cur;
  }
  for (int i = 0; i < K - 1; ++i) st[i] = __float2bfloat16(hist[3 - (K - 1) + i]);
}

__global__ void gdn_gates_kernel(const bf16* __restrict__ a, long long lda, const bf16* __restrict__ b, long long ldb,
                                 const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ g,
                                 float* __restrict__ beta, int tokens, int hv) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * hv) return;
  const int t = idx / hv, h = idx % hv;
  const float x = __bfloat162float(a[t * lda + h]) + dt_bias[h];
  const float sp = x > 20.f ? x : log1pf(expf(x));
  g[idx] = -expf(a_log[h]) * sp;
  beta[idx] = 1.f / (1.f + expf(-__bfloat162float(b[t * ldb + h])));
}

constexpr int TOK_STAGE = 16;
constexpr int GDN_COLS = 32;  // state columns per CTA (4 threads per column)

// q, k: [T, Hk, DK] (row stride ld_qk elements, heads contiguous); v: [T, Hv, DV]; out [T, Hv, DV].
// CTA = (32 state columns of one value head, sequence); four lanes of a warp share a column,
// each holding a quarter of its DK state elements in registers.  Tokens are staged 16 at a
// time through two shared-memory buffers: the raw q/k/v/g/beta of the next 16 tokens are
// loaded into registers before the current 16 are processed and normalised into the other
// buffer afterwards, so global latency overlaps the recurrence and there is one barrier per
// 16 tokens.  The kernel is bound by FMA issue (3 x Dk x Dv multiply-adds per token and head
// on the CUDA cores): measured variants with two columns per thread and fp16 staging moved
// shared-memory traffic down 4x without changing the time.
// XW (steps of at most four tokens per sequence: decode and verify rows): a warp owns one quarter of Dk for all 32 columns
// of the CTA, so each of its state loads and stores is one 128-byte row and its shared-memory reads of k and q are
// broadcasts; the four quarters meet through shared memory with two barriers per token instead of two shuffles.
template <int DK, bool PIPE, bool XW>
__global__ void __launch_bounds__(128) gdn_recurrent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, long long ld_qk,
                                                             const bf16* __restrict__ v, long long ld_v, const float* __restrict__ g,
                                                             const float* __restrict__ beta, float* __restrict__ state, bf16* __restrict__ out,
                                                             const int* __restrict__ q_indptr, const int* __restrict__ slots, int hk, int hv,
                                                             int dv, int col_groups, int skip_len) {
  constexpr int QK = DK / 4;    // state elements per thread
  constexpr int QS = QK + 4;    // padded quarter stride in shared memory: the four quarters land in different banks
  constexpr int QL = DK / 32;   // q / k elements per lane when a warp holds one token
  constexpr int ST = XW ? 4 : TOK_STAGE;  // tokens per stage: short steps keep shared memory small, so more CTAs stay resident
  constexpr int NBUF = PIPE ? 2 : 1;      // only the prefetching variant needs a second stage buffer
  constexpr int TPW = ST / 4;             // tokens per warp and stage
  constexpr int VPT = ST * GDN_COLS / 128;
  __shared__ __align__(16) float sq[NBUF][ST][4 * QS], sk[NBUF][ST][4 * QS];
  __shared__ float sv[NBUF][ST][GDN_COLS], sg[NBUF][ST], sb[NBUF][ST];
  __shared__ float red_kv[4][GDN_COLS], red_o[4][GDN_COLS];
  const int h = blockIdx.x / col_groups, cg = blockIdx.x % col_groups, b = blockIdx.y;
  const int slot = slots[b];
  const int q0 = q_indptr[b], q1 = q_indptr[b + 1];
  if (q1 == q0 || slot < 0) return;
  if (skip_len > 0 && q1 - q0 >= skip_len) return;  // long sequences belong to the chunk-wise kernel
  const int kh = h / (hv / hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qtr = XW ? warp : (tid & 3), lc = XW ? lane : (tid >> 2), col = cg * GDN_COLS + lc;
  const bool owner = col < dv;
  float* S = state + (((long long)slot * hv + h) * DK) * dv;  // [DK][dv], v contiguous
  float s_col[QK];
#pragma unroll
  for (int i = 0; i < QK; ++i) s_col[i] = owner ? S[(long long)(qtr * QK + i) * dv + col] : 0.f;
  const float q_scale = rsqrtf((float)DK);

  // raw next-stage values held in registers between fetch and commit
  float rq[TPW][QL], rk[TPW][QL], rv[VPT], rg = 0.f, rb = 0.f;
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int jj = 0; jj < TPW; ++jj) {
      const int j = warp + 4 * jj;
      const bf16* qp = q + (long long)(t0 + j) * ld_qk + (long long)kh * DK;
      const bf16* kp = k + (long long)(t0 + j) * ld_qk + (long long)kh * DK;
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        rq[jj][i] = j < nt ? __bfloat162float(qp[lane + 32 * i]) : 0.f;
        rk[jj][i] = j < nt ? __bfloat162float(kp[lane + 32 * i]) : 0.f;
      }
    }
#pragma unroll
    for (int x = 0; x < VPT; ++x) {
      const int idx = tid + 128 * x, j = idx / GDN_COLS, d = cg * GDN_COLS + idx % GDN_COLS;
      rv[x] = (j < nt && d < dv) ? __bfloat162float(v[(long long)(t0 + j) * ld_v + (long long)h * dv + d]) : 0.f;
    }
    if (tid < nt) {
      rg = expf(g[(long long)(t0 + tid) * hv + h]);
      rb = beta[(long long)(t0 + tid) * hv + h];
    }
  };
  auto commit = [&](int buf, int nt) {
#pragma unroll
    for (int jj = 0; jj < TPW; ++jj) {
      const int j = warp + 4 * jj;
      float qs = 0.f, ks = 0.f;
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        qs += rq[jj][i] * rq[jj][i];
        ks += rk[jj][i] * rk[jj][i];
      }
      qs = warp_sum(qs);
      ks = warp_sum(ks);
      const float qn = rsqrtf(qs + 1e-6f) * q_scale, kn = rsqrtf(ks + 1e-6f);
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        const int e = lane + 32 * i;
        sq[buf][j][(e / QK) * QS + (e % QK)] = rq[jj][i] * qn;
        sk[buf][j][(e / QK) * QS + (e % QK)] = rk[jj][i] * kn;
      }
    }
#pragma unroll
    for (int x = 0; x < VPT; ++x) {
      const int idx = tid + 128 * x;
      sv[buf][idx / GDN_COLS][idx % GDN_COLS] = rv[x];
    }
    if (tid < nt) {
      sg[buf][tid] = rg;
      sb[buf][tid] = rb;
    }
  };
  auto process = [&](int buf, int t0, int nt) {
    for (int j = 0; j < nt; ++j) {
      const float decay = sg[buf][j];
      const float4* kq = reinterpret_cast<const float4*>(&sk[buf][j][qtr * QS]);
      const float4* qq = reinterpret_cast<const float4*>(&sq[buf][j][qtr * QS]);
      // four independent accumulation chains per dot product
      float4 kv4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < QK / 4; ++i) {
        const float4 kk = kq[i];
        s_col[4 * i + 0] *= decay;
        s_col[4 * i + 1] *= decay;
        s_col[4 * i + 2] *= decay;
        s_col[4 * i + 3] *= decay;
        kv4.x += s_col[4 * i + 0] * kk.x;
        kv4.y += s_col[4 * i + 1] * kk.y;
        kv4.z += s_col[4 * i + 2] * kk.z;
        kv4.w += s_col[4 * i + 3] * kk.w;
      }
      float kv = (kv4.x + kv4.y) + (kv4.z + kv4.w);
      if (XW) {
        red_kv[qtr][lc] = kv;
        __syncthreads();
        kv = (red_kv[0][lc] + red_kv[1][lc]) + (red_kv[2][lc] + red_kv[3][lc]);
      } else {
        kv += __shfl_xor_sync(0xffffffffu, kv, 1);
        kv += __shfl_xor_sync(0xffffffffu, kv, 2);
      }
      const float delta = (sv[buf][j][lc] - kv) * sb[buf][j];
      float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < QK / 4; ++i) {
        const float4 kk = kq[i], qv = qq[i];
        s_col[4 * i + 0] += kk.x * delta;
        s_col[4 * i + 1] += kk.y * delta;
        s_col[4 * i + 2] += kk.z * delta;
        s_col[4 * i + 3] += kk.w * delta;
        o4.x += s_col[4 * i + 0] * qv.x;
        o4.y += s_col[4 * i + 1] * qv.y;
        o4.z += s_col[4 * i + 2] * qv.z;
        o4.w += s_col[4 * i + 3] * qv.w;
      }
      float o = (o4.x + o4.y) + (o4.z + o4.w);
      if (XW) {
        red_o[qtr][lc] = o;
        __syncthreads();  // also orders this token's reads of red_kv before the next token's writes
        o = (red_o[0][lc] + red_o[1][lc]) + (red_o[2][lc] + red_o[3][lc]);
      } else {
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
      }
      if (owner && qtr == 0) out[((long long)(t0 + j) * hv + h) * dv + col] = __float2bfloat16(o);
    }
  };

  if (PIPE) {
    fetch(q0, min(ST, q1 - q0));
    commit(0, min(ST, q1 - q0));
    __syncthreads();
    int buf = 0;
    for (int t0 = q0; t0 < q1; t0 += ST, buf ^= 1) {
      const int nt = min(ST, q1 - t0);
      const int nnext = min(ST, q1 - (t0 + ST));
      if (nnext > 0) fetch(t0 + ST, nnext);
      process(buf, t0, nt);
      if (nnext > 0) commit(buf ^ 1, nnext);
      __syncthreads();
    }
  } else {
    // decode and other short steps: no prefetch registers, more CTAs per SM for the state stream
    for (int t0 = q0; t0 < q1; t0 += ST) {
      const int nt = min(ST, q1 - t0);
      fetch(t0, nt);
      commit(0, nt);
      __syncthreads();
      process(0, t0, nt);
      __syncthreads();
    }
  }
  if (owner) {
#pragma unroll
    for (int i = 0; i < QK; ++i) S[(long long)(qtr * QK + i) * dv + col] = s_col[i];
  }
}

}  // namespace

extern "C" int pg_gdn_conv1d(const void* x, long long ldx, const void* w, void* state, void* out, long long ldo, const void* q_indptr,
                             const void* slots, int num_seqs, int channels, int K, long long state_slot_stride, cudaStream_t stream) {
  PG_REQUIRE(K >= 2 && K <= 4, "gdn_conv1d: kernel size %d not supported (2..4)", K);
  if (num_seqs == 0) return PG_OK;
  dim3 grid((channels + 127) / 128, num_seqs);
  gdn_conv1d_kernel<<<grid, 128, 0, stream>>>((const bf16*)x, ldx, (const bf16*)w, (bf16*)state, (bf16*)out, ldo, (const int*)q_indptr,
                                             (const int*)slots, channels, K, state_slot_stride);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_gdn_gates(const void* a, long long lda, const void* b, long long ldb, const void* a_log, const void* dt_bias, void* g, void* beta,
                            int tokens, int hv, cudaStream_t stream) {
  if (tokens == 0) return PG_OK;
  gdn_gates_kernel<<<(tokens * hv + 255) / 256, 256, 0, stream>>>((const bf16*)a, lda, (const bf16*)b, ldb, (const float*)a_log,
                                                                 (const float*)dt_bias, (float*)g, (float*)beta, tokens, hv);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_gdn_recurrent(const void* q, const void* k, long long ld_qk, const void* v, long long ld_v, const void* g, const void* beta,
                                void* state, void* out, const void* q_indptr, const void* slots, int num_seqs, int hk, int hv, int dk, int dv,
                                int max_q_len, int skip_len, cudaStream_t stream) {
  // skip_len > 0: sequences of at least that many tokens are left to pg_gdn_chunked
  // steps longer than one stage of 16 tokens use the variant that prefetches the next stage
  const bool long_steps = max_q_len > 16;
  PG_REQUIRE(dv <= 128 && hv % hk == 0, "gdn_recurrent: dv=%d must be <= 128 and hv %% hk == 0", dv);
  if (num_seqs == 0) return PG_OK;
  const int col_groups = (dv + GDN_COLS - 1) / GDN_COLS;
  dim3 grid(hv * col_groups, num_seqs);
  const bool few = max_q_len <= 4;  // decode and verify rows: the row-coalesced mapping
#define PG_GDN_ARGS                                                                                                                       \
  (const bf16*)q, (const bf16*)k, ld_qk, (const bf16*)v, ld_v, (const float*)g, (const float*)beta, (float*)state, (bf16*)out,           \
      (const int*)q_indptr, (const int*)slots, hk, hv, dv, col_groups, skip_len
#define PG_GDN_LAUNCH(DKV)                                                               \
  do {                                                                                   \
    if (long_steps)                                                                      \
      gdn_recurrent_kernel<DKV, true, false><<<grid, 128, 0, stream>>>(PG_GDN_ARGS);     \
    else if (few)                                                                        \
      gdn_recurrent_kernel<DKV, false, true><<<grid, 128, 0, stream>>>(PG_GDN_ARGS);     \
    else                                                                                 \
      gdn_recurrent_kernel<DKV, false, false><<<grid, 128, 0, stream>>>(PG_GDN_ARGS);    \
  } while (0)
  if (dk == 128)
    PG_GDN_LAUNCH(128);
  else if (dk == 64)
    PG_GDN_LAUNCH(64);
  else if (dk == 32)
    PG_GDN_LAUNCH(32);
  else {
    pg_set_error("gdn_recurrent: dk=%d not supported (32, 64, 128)", dk);
    return PG_ERR_UNSUPPORTED;
  }
#undef PG_GDN_LAUNCH
#undef PG_GDN_ARGS
  PG_LAUNCH_CHECK();
  return PG_OK;
}
