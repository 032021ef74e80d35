// Gated DeltaNet kernels (Qwen3.5 linear-attention layers).
//
//  * gdn_conv1d: causal depthwise conv (kernel <= 4) + SiLU over ragged sequences with a
//    carried [C, K-1] input history per sequence slot (prefill and decode in one kernel).
//  * gdn_gates: g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b).
//  * gdn_recurrent: the gated delta rule.  One CTA per (sequence, value head); thread v
//    owns column v of the f32 state S[Dk, Dv] in registers, so S^T k, the rank-1 update
//    and S^T q are thread-local dot products over Dk with no cross-thread reduction; the
//    CTA stages 8 tokens of (q, k, v, g, beta) in shared memory per barrier.  A decode
//    step is one pass over the 64 KiB state (read + write: HBM bound); a prefill chunk
//    walks its tokens in order with the state resident in registers.
//
// Functional parity with pegainfer-kernels/csrc/qwen35/conv1d.cu:19-165,
// gated_delta_rule.cu:28-347 and the chunk-wise Triton prefill pipeline
// (tools/triton/gated_delta_rule_chunkwise_kernels.py), whose result equals this
// recurrence.
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

constexpr int TOK_STAGE = 8;

// q, k: [T, Hk, DK] (row stride ld_qk elements, heads contiguous); v: [T, Hv, DV]; out [T, Hv, DV].
template <int DK>
__global__ void __launch_bounds__(128) gdn_recurrent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, long long ld_qk,
                                                             const bf16* __restrict__ v, long long ld_v, const float* __restrict__ g,
                                                             const float* __restrict__ beta, float* __restrict__ state, bf16* __restrict__ out,
                                                             const int* __restrict__ q_indptr, const int* __restrict__ slots, int hk, int hv,
                                                             int dv) {
  __shared__ float sq[TOK_STAGE][DK], sk[TOK_STAGE][DK];
  __shared__ float sv[TOK_STAGE][128], sg[TOK_STAGE], sb[TOK_STAGE];
  const int h = blockIdx.x, b = blockIdx.y;
  const int slot = slots[b];
  const int q0 = q_indptr[b], q1 = q_indptr[b + 1];
  if (q1 == q0 || slot < 0) return;
  const int kh = h / (hv / hk);
  const int tid = threadIdx.x;
  const bool owner = tid < dv;
  float* S = state + (((long long)slot * hv + h) * DK) * dv;  // [DK][dv], v contiguous
  float s_col[DK];
  if (owner) {
#pragma unroll
    for (int i = 0; i < DK; ++i) s_col[i] = S[(long long)i * dv + tid];
  }
  const float q_scale = rsqrtf((float)DK);
  for (int t0 = q0; t0 < q1; t0 += TOK_STAGE) {
    const int nt = min(TOK_STAGE, q1 - t0);
    __syncthreads();
    // stage nt tokens: each warp normalises q and k of tokens w, w+4
    const int warp = tid >> 5, lane = tid & 31;
    for (int j = warp; j < nt; j += 4) {
      const bf16* qp = q + (long long)(t0 + j) * ld_qk + (long long)kh * DK;
      const bf16* kp = k + (long long)(t0 + j) * ld_qk + (long long)kh * DK;
      float qs = 0.f, ks = 0.f;
      for (int i = lane; i < DK; i += 32) {
        const float a = __bfloat162float(qp[i]), c = __bfloat162float(kp[i]);
        sq[j][i] = a;
        sk[j][i] = c;
        qs += a * a;
        ks += c * c;
      }
      qs = warp_sum(qs);
      ks = warp_sum(ks);
      const float qn = rsqrtf(qs + 1e-12f) * q_scale, kn = rsqrtf(ks + 1e-12f);
      for (int i = lane; i < DK; i += 32) {
        sq[j][i] *= qn;
        sk[j][i] *= kn;
      }
      if (lane == 0) {
        sg[j] = expf(g[(long long)(t0 + j) * hv + h]);
        sb[j] = beta[(long long)(t0 + j) * hv + h];
      }
    }
    for (int idx = tid; idx < nt * dv; idx += 128) {
      const int j = idx / dv, d = idx % dv;
      sv[j][d] = __bfloat162float(v[(long long)(t0 + j) * ld_v + (long long)h * dv + d]);
    }
    __syncthreads();
    if (owner) {
      for (int j = 0; j < nt; ++j) {
        const float decay = sg[j];
        float kv = 0.f;
#pragma unroll
        for (int i = 0; i < DK; ++i) {
          s_col[i] *= decay;
          kv += s_col[i] * sk[j][i];
        }
        const float delta = (sv[j][tid] - kv) * sb[j];
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DK; ++i) {
          s_col[i] += sk[j][i] * delta;
          o += s_col[i] * sq[j][i];
        }
        out[((long long)(t0 + j) * hv + h) * dv + tid] = __float2bfloat16(o);
      }
    }
  }
  if (owner) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[(long long)i * dv + tid] = s_col[i];
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
                                cudaStream_t stream) {
  PG_REQUIRE(dv <= 128 && hv % hk == 0, "gdn_recurrent: dv=%d must be <= 128 and hv %% hk == 0", dv);
  if (num_seqs == 0) return PG_OK;
  dim3 grid(hv, num_seqs);
#define PG_GDN_LAUNCH(DKV)                                                                                                                  \
  gdn_recurrent_kernel<DKV><<<grid, 128, 0, stream>>>((const bf16*)q, (const bf16*)k, ld_qk, (const bf16*)v, ld_v, (const float*)g,        \
                                                      (const float*)beta, (float*)state, (bf16*)out, (const int*)q_indptr, (const int*)slots, \
                                                      hk, hv, dv)
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
  PG_LAUNCH_CHECK();
  return PG_OK;
}
