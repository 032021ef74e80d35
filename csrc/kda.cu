// Kernels of the KDA + latent-MoE model line (Kimi-K3 shape).
//
//  * kda_recurrent: the delta rule with a decay per key channel.  Per token and head,
//      dec[d] = exp(lower * sigmoid(exp(A_log[h]) * (f[d] + dt_bias[h, d])))   (lower < 0, so dec in (e^lower, 1))
//      S      = S * dec (rows of S[Dk, Dv] scaled)        kv = S^T k
//      S     += k (x) ((v - kv) * sigmoid(b))             out = S^T q
//    with q and k L2-normalised (q also times Dk^-0.5).  The gate arithmetic runs inside the kernel, so the
//    step needs no separate gate launch.  The state layout and the thread mapping are those of the scalar-decay
//    rule in gdn.cu: a CTA takes 32 columns of one (sequence, head), four lanes share a column and each keeps a
//    quarter of its Dk elements in registers; a stage of 8 tokens is normalised into shared memory, then
//    walked in order.  A decode step is one pass over the state (read + write).
//  * attnres_mix: the attention-residual mix.  Every token keeps up to `cap` snapshot rows of its own residual
//    stream; a mix scores each of the first nb snapshots and the current row with
//    dot(x / rms(x), score_w) and returns the softmax-weighted sum of the un-normalised rows.
//
// Functional parity with pegainfer-k3/kernels/tilelang_defs.py:67-139 (attnres_scores / attnres_mix) and
// :304-410 (kda_core) and pegainfer-kernels/csrc/k3/k3_flash_kda.cu (chunked prefill of the same rule).
#include "api.h"
#include "common.cuh"

namespace {

constexpr int KDA_STAGE = 8;
constexpr int KDA_COLS = 32;

// XW = false: four adjacent lanes share a state column and reduce with shuffles (prompt chunks: no barrier per token).
// XW = true: a warp owns one quarter of Dk for all 32 columns, so every state load and store of a warp is one 128-byte row
// and the shared-memory reads of k, q and the decays are broadcasts; the four quarters meet through shared memory with two
// barriers per token (decode rows and other steps of a few tokens).
template <int DK, bool XW>
__global__ void __launch_bounds__(128) kda_recurrent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, long long ld,
                                                             const bf16* __restrict__ f, long long ldf, const bf16* __restrict__ b, long long ldb,
                                                             const float* __restrict__ a_log, const float* __restrict__ dt_bias, float lower,
                                                             float* __restrict__ state, bf16* __restrict__ out, const int* __restrict__ q_indptr,
                                                             const int* __restrict__ slots, int heads, int dv, int col_groups) {
  constexpr int QK = DK / 4;   // state elements per thread
  constexpr int QS = QK + 4;   // padded quarter stride: the four quarters land in different banks
  constexpr int QL = DK / 32;  // elements per lane when a warp holds one token
  __shared__ __align__(16) float sq[KDA_STAGE][4 * QS], sk[KDA_STAGE][4 * QS], sd[KDA_STAGE][4 * QS];
  __shared__ float sv[KDA_STAGE][KDA_COLS], sb[KDA_STAGE];
  __shared__ float red_kv[4][KDA_COLS], red_o[4][KDA_COLS];
  const int h = blockIdx.x / col_groups, cg = blockIdx.x % col_groups, seq = blockIdx.y;
  const int slot = slots[seq];
  const int q0 = q_indptr[seq], q1 = q_indptr[seq + 1];
  if (q1 == q0 || slot < 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qtr = XW ? warp : (tid & 3), lc = XW ? lane : (tid >> 2), col = cg * KDA_COLS + lc;
  const bool owner = col < dv;
  float* S = state + (((long long)slot * heads + h) * DK) * dv;  // [DK][dv], v contiguous
  // Shuffle mapping: a thread's own elements sit DK / 4 rows apart, so a warp reads 32-byte pieces of four rows.  Staging
  // the CTA's slice through shared memory instead was measured slower (200 us against 111 us for 32 decode rows of 96
  // heads: the extra 17 KB per CTA costs resident CTAs); the XW mapping reads whole rows without it (86 us).
  float s_col[QK];
#pragma unroll
  for (int i = 0; i < QK; ++i) s_col[i] = owner ? S[(long long)(qtr * QK + i) * dv + col] : 0.f;
  const float q_scale = rsqrtf((float)DK);
  const float a = __expf(a_log[h]);

  for (int t0 = q0; t0 < q1; t0 += KDA_STAGE) {
    const int nt = min(KDA_STAGE, q1 - t0);
    // stage: each warp normalises two tokens' q and k and turns the gate row into decays
    for (int j = warp; j < nt; j += 4) {
      const long long row = (long long)(t0 + j);
      const bf16* qp = q + row * ld + (long long)h * DK;
      const bf16* kp = k + row * ld + (long long)h * DK;
      const bf16* fp = f + row * ldf + (long long)h * DK;
      float rq[QL], rk[QL], qs = 0.f, ks = 0.f;
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        rq[i] = __bfloat162float(qp[lane + 32 * i]);
        rk[i] = __bfloat162float(kp[lane + 32 * i]);
        qs += rq[i] * rq[i];
        ks += rk[i] * rk[i];
      }
      qs = warp_sum(qs);
      ks = warp_sum(ks);
      const float qn = rsqrtf(qs + 1e-6f) * q_scale, kn = rsqrtf(ks + 1e-6f);
#pragma unroll
      for (int i = 0; i < QL; ++i) {
        const int e = lane + 32 * i, at = (e / QK) * QS + (e % QK);
        const float raw = __bfloat162float(fp[e]) + dt_bias[h * DK + e];
        sq[j][at] = rq[i] * qn;
        sk[j][at] = rk[i] * kn;
        sd[j][at] = __expf(lower / (1.f + __expf(-a * raw)));
      }
    }
    for (int idx = tid; idx < nt * KDA_COLS; idx += 128) {
      const int j = idx / KDA_COLS, d = cg * KDA_COLS + idx % KDA_COLS;
      sv[j][idx % KDA_COLS] = d < dv ? __bfloat162float(v[(long long)(t0 + j) * ld + (long long)h * dv + d]) : 0.f;
    }
    if (tid < nt) sb[tid] = 1.f / (1.f + __expf(-__bfloat162float(b[(long long)(t0 + tid) * ldb + h])));
    __syncthreads();
    for (int j = 0; j < nt; ++j) {
      const float4* kq = reinterpret_cast<const float4*>(&sk[j][qtr * QS]);
      const float4* qq = reinterpret_cast<const float4*>(&sq[j][qtr * QS]);
      const float4* dq = reinterpret_cast<const float4*>(&sd[j][qtr * QS]);
      float4 kv4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < QK / 4; ++i) {
        const float4 kk = kq[i], dd = dq[i];
        s_col[4 * i + 0] *= dd.x;
        s_col[4 * i + 1] *= dd.y;
        s_col[4 * i + 2] *= dd.z;
        s_col[4 * i + 3] *= dd.w;
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
      const float delta = (sv[j][lc] - kv) * sb[j];
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
      if (owner && qtr == 0) out[((long long)(t0 + j) * heads + h) * dv + col] = __float2bfloat16(o);
    }
    __syncthreads();
  }
  if (owner) {
#pragma unroll
    for (int i = 0; i < QK; ++i) S[(long long)(qtr * QK + i) * dv + col] = s_col[i];
  }
}

constexpr int ATTNRES_MAX = 16;  // candidates of one mix (snapshots + the current row)

// One CTA of 256 threads per token.  Pass 1: sum of squares and dot with score_w for every candidate; pass 2: softmax of
// the scores and the weighted sum (the rows come back from L1 / L2).
__global__ void __launch_bounds__(256) attnres_mix_kernel(const bf16* __restrict__ cur, long long ld_cur, const bf16* __restrict__ snaps, long long ld_tok,
                                                           const float* __restrict__ score_w, bf16* __restrict__ out, long long ld_out, int nb, int hidden,
                                                           float eps) {
  PG_PDL_ENTRY();
  __shared__ float red[2][ATTNRES_MAX][8];
  __shared__ float prob[ATTNRES_MAX];
  const long long t = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nvec = hidden / 8;
  const int nc = nb + 1;
  auto row = [&](int c) { return c < nb ? snaps + t * ld_tok + (long long)c * hidden : cur + t * ld_cur; };
  for (int c = 0; c < nc; ++c) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(row(c));
    float ss = 0.f, dot = 0.f;
    for (int i = tid; i < nvec; i += 256) {
      float x[8];
      unpack8(xr[i], x);
      const float4 w0 = reinterpret_cast<const float4*>(score_w)[2 * i], w1 = reinterpret_cast<const float4*>(score_w)[2 * i + 1];
      ss += x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3] + x[4] * x[4] + x[5] * x[5] + x[6] * x[6] + x[7] * x[7];
      dot += x[0] * w0.x + x[1] * w0.y + x[2] * w0.z + x[3] * w0.w + x[4] * w1.x + x[5] * w1.y + x[6] * w1.z + x[7] * w1.w;
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    if (lane == 0) red[0][c][warp] = ss, red[1][c][warp] = dot;
  }
  __syncthreads();
  if (tid == 0) {
    float sc[ATTNRES_MAX], mx = -1e30f, den = 0.f;
    for (int c = 0; c < nc; ++c) {
      float ss = 0.f, dot = 0.f;
      for (int w = 0; w < 8; ++w) ss += red[0][c][w], dot += red[1][c][w];
      sc[c] = dot * rsqrtf(ss / (float)hidden + eps);
      mx = fmaxf(mx, sc[c]);
    }
    for (int c = 0; c < nc; ++c) den += (sc[c] = __expf(sc[c] - mx));
    for (int c = 0; c < nc; ++c) prob[c] = sc[c] / den;
  }
  __syncthreads();
  for (int i = tid; i < nvec; i += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < nc; ++c) {
      float x[8];
      unpack8(reinterpret_cast<const bf16x8*>(row(c))[i], x);
      const float p = prob[c];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += p * x[j];
    }
    reinterpret_cast<bf16x8*>(out + t * ld_out)[i] = pack8(acc);
  }
}

}  // namespace

extern "C" int pg_kda_recurrent(const void* q, const void* k, const void* v, long long ld, const void* f, long long ldf, const void* b, long long ldb,
                                const void* a_log, const void* dt_bias, float lower, void* state, void* out, const void* q_indptr, const void* slots,
                                int num_seqs, int heads, int dk, int dv, int max_q_len, cudaStream_t stream) {
  PG_REQUIRE(dv <= 128 && lower < 0.f, "kda_recurrent: dv=%d must be <= 128 and the decay lower bound %f negative", dv, (double)lower);
  if (num_seqs == 0) return PG_OK;
  const int col_groups = (dv + KDA_COLS - 1) / KDA_COLS;
  dim3 grid(heads * col_groups, num_seqs);
  const bool few = max_q_len <= 4;  // decode rows and verify steps: the row-coalesced mapping
#define PG_KDA_ARGS                                                                                                                              \
  (const bf16*)q, (const bf16*)k, (const bf16*)v, ld, (const bf16*)f, ldf, (const bf16*)b, ldb, (const float*)a_log, (const float*)dt_bias, lower, \
      (float*)state, (bf16*)out, (const int*)q_indptr, (const int*)slots, heads, dv, col_groups
#define PG_KDA_LAUNCH(DKV)                                                     \
  do {                                                                         \
    if (few)                                                                   \
      kda_recurrent_kernel<DKV, true><<<grid, 128, 0, stream>>>(PG_KDA_ARGS);  \
    else                                                                       \
      kda_recurrent_kernel<DKV, false><<<grid, 128, 0, stream>>>(PG_KDA_ARGS); \
  } while (0)
  if (dk == 128)
    PG_KDA_LAUNCH(128);
  else if (dk == 64)
    PG_KDA_LAUNCH(64);
  else if (dk == 32)
    PG_KDA_LAUNCH(32);
  else {
    pg_set_error("kda_recurrent: dk=%d not supported (32, 64, 128)", dk);
    return PG_ERR_UNSUPPORTED;
  }
#undef PG_KDA_LAUNCH
#undef PG_KDA_ARGS
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_attnres_mix(const void* cur, long long ld_cur, const void* snaps, long long ld_tok, const void* score_w, void* out, long long ld_out,
                              int tokens, int nb, int hidden, float eps, cudaStream_t stream) {
  PG_REQUIRE(nb >= 0 && nb + 1 <= ATTNRES_MAX && hidden % 8 == 0 && ld_cur % 8 == 0 && ld_tok % 8 == 0 && ld_out % 8 == 0,
             "attnres_mix: %d snapshots (at most %d) and a hidden size %d that is a multiple of 8", nb, ATTNRES_MAX - 1, hidden);
  if (tokens == 0) return PG_OK;
  PG_CUDA(launch_pdl(attnres_mix_kernel, dim3(tokens), dim3(256), (size_t)(0), stream, (const bf16*)cur, ld_cur, (const bf16*)snaps, ld_tok,
                     (const float*)score_w, (bf16*)out, ld_out, nb, hidden, eps));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
