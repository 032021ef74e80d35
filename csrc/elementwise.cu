// Memory-bound row kernels: embedding / row gather, RMSNorm (+ fused residual add,
// (1+w) weights, round-before-norm), gated RMSNorm, SwiGLU, and the fused
// QK-RMSNorm + RoPE + paged-KV append that sits between the qkv GEMM and attention.
// All use 16-byte vector accesses; rows must be multiples of 8 bf16 elements.
//
// Functional parity with pegainfer-kernels/csrc/shared/{elementwise.cu:376-497,
// flashinfer_norm.cu:40-312, fused_proj.cu:12-46, norm.cu:19-71, prefill_attention.cu:39-124},
// csrc/qwen35/prefill_attention_hd256.cu:41-326 and paged_attention.cu:287-364 (KV append),
// with an error status word where the reference traps on a bad position.
#include "api.h"
#include "common.cuh"

namespace {

__global__ void gather_rows_kernel(const bf16* __restrict__ table, const int* __restrict__ ids, bf16* __restrict__ out, int rows, int width,
                                   long long table_rows, uint32_t* status) {
  PG_PDL_ENTRY();
  const int t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= table_rows) {
    if (threadIdx.x == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (2u << 8));
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + id * (long long)width);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * width);
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

// dst[i] = src[idx[i]] for 32-bit words (token ids moved between decode steps on the device).
__global__ void gather_words_kernel(const uint32_t* __restrict__ src, const int* __restrict__ idx, uint32_t* __restrict__ dst, int n, int src_len,
                                    uint32_t* status) {
  PG_PDL_ENTRY();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int j = idx[i];
  if (j < 0 || j >= src_len) {
    atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (12u << 8));
    j = 0;
  }
  dst[i] = src[j];
}

// One CTA per row.  MODE 0: y = norm(x).  MODE 1: res += x; y = norm(res).
template <int MODE>
__global__ void __launch_bounds__(256) rms_norm_kernel(const bf16* __restrict__ x, bf16* __restrict__ residual, const bf16* __restrict__ w,
                                                        bf16* __restrict__ y, int width, float eps, int offset, int round_before, long long ldx,
                                                        long long ldr, long long ldy) {
  PG_PDL_ENTRY();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = width / 8;
  constexpr int MAXV = 4;  // register-resident up to 8192 columns with 256 threads
  float vals[MAXV][8];
  float ss = 0.f;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * ldx);
  bf16x8* rr = MODE == 1 ? reinterpret_cast<bf16x8*>(residual + row * ldr) : nullptr;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < nvec) {
      float f[8];
      unpack8(xr[i], f);
      if (MODE == 1) {
        float r[8];
        unpack8(rr[i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
        bf16x8 packed = pack8(f);
        rr[i] = packed;
        if (round_before) unpack8(packed, f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[k][j] = f[j];
        ss += f[j] * f[j];
      }
    }
  }
  // columns beyond the register window (width > 8192): recomputed in a second pass
  for (int i = threadIdx.x + MAXV * 256; i < nvec; i += 256) {
    float f[8];
    unpack8(xr[i], f);
    if (MODE == 1) {
      float r[8];
      unpack8(rr[i], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += r[j];
      bf16x8 packed = pack8(f);
      rr[i] = packed;
      if (round_before) unpack8(packed, f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)width + eps);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * ldy);
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < nvec) {
      float wf[8], o[8];
      unpack8(wr[i], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[k][j] * inv * (offset ? wf[j] + 1.f : wf[j]);
      yr[i] = pack8(o);
    }
  }
  for (int i = threadIdx.x + MAXV * 256; i < nvec; i += 256) {
    float f[8], wf[8], o[8];
    // MODE 1 with round_before re-reads the stored residual (already the rounded sum)
    unpack8(MODE == 1 ? rr[i] : xr[i], f);
    unpack8(wr[i], wf);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = f[j] * inv * (offset ? wf[j] + 1.f : wf[j]);
    yr[i] = pack8(o);
  }
}

// Per (token, head): y = rms_norm(x, w_f32) * silu(gate); one warp per head row.
// act 0: rms_norm(x) * w * silu(gate), rounded once; act 1: bf16(rms_norm(x) * w) * bf16(sigmoid(gate))
__global__ void gated_rms_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate, const float* __restrict__ w, bf16* __restrict__ y,
                                      long long rows, int dim, float eps, int act) {
  PG_PDL_ENTRY();
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const bf16* xr = x + row * dim;
  const bf16* gr = gate + row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    float v = __bfloat162float(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)dim + eps);
  for (int i = lane; i < dim; i += 32) {
    float v = __bfloat162float(xr[i]);
    float g = __bfloat162float(gr[i]);
    if (act == 1) {
      y[row * dim + i] = __float2bfloat16(bf16_round(v * inv * w[i]) * bf16_round(1.f / (1.f + __expf(-g))));
      continue;
    }
    float s = g / (1.f + __expf(-g));
    y[row * dim + i] = __float2bfloat16(v * inv * w[i] * s);
  }
}

// `interleaved` = 0: a row is [gate_0 .. gate_{I-1}, up_0 .. up_{I-1}]; 1: (gate_0, up_0, gate_1, up_1, ...).
// `flags`: bit 0 = gate / up columns interleaved, bit 1 = tanh GELU instead of SiLU on the gate (GeGLU), bit 2 = the
// saturating form 4 tanh(g / 4) sigmoid(g) * 25 tanh(u / 25), rounded once (pegainfer-k3/kernels/tilelang_defs.py:244-262)
__global__ void swiglu_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int rows, int inter, long long ldin, long long ldout, int flags) {
  PG_PDL_ENTRY();
  const int interleaved = flags & 1, gelu = flags & 2, situ = flags & 4;
  const int nvec = inter / 8;
  const long long total = (long long)rows * nvec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx / nvec), i = (int)(idx % nvec);
    float gf[8], uf[8], o[8];
    if (interleaved) {
      const bf16x8* pr = reinterpret_cast<const bf16x8*>(gu + row * ldin) + 2 * i;
      float a[8], b[8];
      unpack8(pr[0], a);
      unpack8(pr[1], b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gf[j] = a[2 * j], uf[j] = a[2 * j + 1];
        gf[4 + j] = b[2 * j], uf[4 + j] = b[2 * j + 1];
      }
    } else {
      const bf16x8* g = reinterpret_cast<const bf16x8*>(gu + row * ldin) + i;
      const bf16x8* u = reinterpret_cast<const bf16x8*>(gu + row * ldin + inter) + i;
      unpack8(*g, gf);
      unpack8(*u, uf);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = gf[j];
      if (situ) {
        o[j] = 4.f * tanhf(0.25f * g) / (1.f + __expf(-g)) * (25.f * tanhf(0.04f * uf[j]));
        continue;
      }
      const float a = gelu ? 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) : g / (1.f + __expf(-g));
      o[j] = bf16_round(a) * uf[j];
    }
    reinterpret_cast<bf16x8*>(out + row * ldout)[i] = pack8(o);
  }
}

__global__ void softcap_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, float cap) {
  PG_PDL_ENTRY();
  const float inv = 1.f / cap;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16(tanhf(__bfloat162float(x[i]) * inv) * cap);
}

__global__ void sigmoid_gate_mul_kernel(bf16* __restrict__ x, const bf16* __restrict__ gate, long long n) {
  PG_PDL_ENTRY();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = __bfloat162float(gate[i]);
    x[i] = __float2bfloat16(__bfloat162float(x[i]) / (1.f + __expf(-g)));
  }
}

// One warp per (token, head) over the fused qkv row.  Heads [0, Hq) are queries,
// [Hq, Hq+Hkv) keys, [Hq+Hkv, Hq+2Hkv) values.
struct RopeParams {
  const bf16* qkv;
  long long ld;
  const bf16* q_w;
  const bf16* k_w;
  const bf16* cos;
  const bf16* sin;
  const int* positions;
  const int* slots;
  bf16* q_out;
  bf16* gate_out;
  bf16* kv;  // [pages, 2, page_size, Hkv, D]
  int tokens, hq, hkv, dim, rot, page_size, max_pos, gated, offset, has_norm;
  int v_norm;  // value rows get a weightless RMSNorm over the head before they are stored
  long long num_slots;
  float eps;
  uint32_t* status;
};

__global__ void __launch_bounds__(128) qk_norm_rope_append_kernel(const RopeParams p) {
  PG_PDL_ENTRY();
  __shared__ float buf[4][256];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  const long long unit = (long long)blockIdx.x * 4 + w;
  if (unit >= (long long)p.tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  const int D = p.dim;
  const int qstride = p.gated ? 2 * D : D;
  const bf16* src;
  int kind;  // 0 q, 1 k, 2 v
  if (h < p.hq) {
    kind = 0;
    src = p.qkv + t * p.ld + (long long)h * qstride;
  } else if (h < p.hq + p.hkv) {
    kind = 1;
    src = p.qkv + t * p.ld + (long long)p.hq * qstride + (long long)(h - p.hq) * D;
  } else {
    kind = 2;
    src = p.qkv + t * p.ld + (long long)p.hq * qstride + (long long)(h - p.hq) * D;  // keys then values are contiguous
  }
  long long slot = p.slots[t];
  if (kind != 0 && (slot < 0 || slot >= p.num_slots)) {
    if (lane == 0) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (3u << 8));
    return;
  }
  const long long page = slot / p.page_size, off = slot % p.page_size;
  if (kind == 2) {
    bf16* dst = p.kv + (((page * 2 + 1) * p.page_size + off) * p.hkv + (h - p.hq - p.hkv)) * D;
    if (p.v_norm) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) {
        const float v = __bfloat162float(src[i]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + p.eps);
      for (int i = lane; i < D; i += 32) dst[i] = __float2bfloat16(__bfloat162float(src[i]) * inv);
      return;
    }
    for (int i = lane; i < D / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  int pos = p.positions[t];
  if (pos < 0 || pos >= p.max_pos) {
    if (lane == 0) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (4u << 8));
    pos = pos < 0 ? 0 : p.max_pos - 1;
  }
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float v = __bfloat162float(src[i]);
    buf[w][i] = v;
    ss += v * v;
  }
  if (p.has_norm) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    const bf16* nw = kind == 0 ? p.q_w : p.k_w;
    for (int i = lane; i < D; i += 32) {
      float wv = __bfloat162float(nw[i]);
      buf[w][i] = bf16_round(buf[w][i] * inv * (p.offset ? wv + 1.f : wv));
    }
  }
  __syncwarp();
  bf16* dst;
  if (kind == 0)
    dst = p.q_out + ((long long)t * p.hq + h) * D;
  else
    dst = p.kv + (((page * 2 + 0) * p.page_size + off) * p.hkv + (h - p.hq)) * D;
  const int half = p.rot / 2;
  const bf16* cs = p.cos + (long long)pos * half;
  const bf16* sn = p.sin + (long long)pos * half;
  for (int i = lane; i < D; i += 32) {
    float o;
    if (i < half) {
      o = buf[w][i] * __bfloat162float(cs[i]) - buf[w][i + half] * __bfloat162float(sn[i]);
    } else if (i < p.rot) {
      o = buf[w][i] * __bfloat162float(cs[i - half]) + buf[w][i - half] * __bfloat162float(sn[i - half]);
    } else {
      o = buf[w][i];
    }
    dst[i] = __float2bfloat16(o);
  }
  if (kind == 0 && p.gated) {
    bf16* g = p.gate_out + ((long long)t * p.hq + h) * D;
    for (int i = lane; i < D; i += 32) g[i] = src[D + i];
  }
}

// Same operation for head dims whose 32 lanes each hold VEC = D / 32 contiguous elements (one 4-, 8- or 16-byte access
// per lane and row, no shared memory): the rotation partner of a lane is lane ^ (rot / 2 / VEC), which needs
// rot / 2 to be a multiple of VEC and rot / 2 / VEC a power of two (full rotary of 64 / 128 / 256, a quarter of 256).
// A warp takes ROPE_G consecutive heads of one token: their rows are loaded together (independent loads in flight), and the
// token's slot, position and cos / sin row are read once for all of them.
constexpr int ROPE_G = 8;
template <int VEC>
__global__ void __launch_bounds__(128) qk_norm_rope_append_vec_kernel(const RopeParams p) {
  PG_PDL_ENTRY();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.hq + 2 * p.hkv;
  const int groups = (heads + ROPE_G - 1) / ROPE_G;
  const long long unit = (long long)blockIdx.x * 4 + w;
  if (unit >= (long long)p.tokens * groups) return;
  const int t = (int)(unit / groups), h0 = (int)(unit % groups) * ROPE_G;
  constexpr int D = VEC * 32;
  const int qstride = p.gated ? 2 * D : D;
  struct alignas(VEC * 2) Pack {
    bf16 v[VEC];
  };
  const bf16* row = p.qkv + t * p.ld;
  auto src_of = [&](int h) { return h < p.hq ? row + (long long)h * qstride : row + (long long)p.hq * qstride + (long long)(h - p.hq) * D; };
  Pack in[ROPE_G];
#pragma unroll
  for (int g = 0; g < ROPE_G; ++g)
    if (h0 + g < heads) in[g] = *reinterpret_cast<const Pack*>(src_of(h0 + g) + lane * VEC);
  long long slot = p.slots[t];
  const bool slot_ok = slot >= 0 && slot < p.num_slots;
  if (!slot_ok && h0 + ROPE_G > p.hq && lane == 0) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (3u << 8));
  const long long page = slot / p.page_size, off = slot % p.page_size;
  int pos = p.positions[t];
  if (pos < 0 || pos >= p.max_pos) {
    if (lane == 0 && h0 < p.hq + p.hkv) atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (4u << 8));
    pos = pos < 0 ? 0 : p.max_pos - 1;
  }
  const int half = p.rot / 2, half_lanes = half / VEC;
  const bool rotated = lane < 2 * half_lanes;
  const bool low = lane < half_lanes;
  const int e0 = (low ? lane : lane - half_lanes) * VEC;  // index into the cos / sin row (valid when rotated)
  float cs[VEC], sn[VEC];
  if (rotated) {
    const Pack c = *reinterpret_cast<const Pack*>(p.cos + (long long)pos * half + e0);
    const Pack s2 = *reinterpret_cast<const Pack*>(p.sin + (long long)pos * half + e0);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      cs[i] = __bfloat162float(c.v[i]);
      sn[i] = low ? -__bfloat162float(s2.v[i]) : __bfloat162float(s2.v[i]);
    }
  }
  float qw[VEC], kw[VEC];
  if (p.has_norm) {
    const Pack a = *reinterpret_cast<const Pack*>(p.q_w + lane * VEC), b2 = *reinterpret_cast<const Pack*>(p.k_w + lane * VEC);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      qw[i] = __bfloat162float(a.v[i]) + (p.offset ? 1.f : 0.f);
      kw[i] = __bfloat162float(b2.v[i]) + (p.offset ? 1.f : 0.f);
    }
  }
#pragma unroll
  for (int g = 0; g < ROPE_G; ++g) {
    const int h = h0 + g;
    if (h >= heads) break;
    const int kind = h < p.hq ? 0 : h < p.hq + p.hkv ? 1 : 2;
    if (kind != 0 && !slot_ok) continue;
    if (kind == 2) {
      bf16* dst = p.kv + (((page * 2 + 1) * p.page_size + off) * p.hkv + (h - p.hq - p.hkv)) * D;
      if (p.v_norm) {
        float vv[VEC], ss = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          vv[i] = __bfloat162float(in[g].v[i]);
          ss += vv[i] * vv[i];
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + p.eps);
        Pack vo;
#pragma unroll
        for (int i = 0; i < VEC; ++i) vo.v[i] = __float2bfloat16(vv[i] * inv);
        *reinterpret_cast<Pack*>(dst + lane * VEC) = vo;
        continue;
      }
      *reinterpret_cast<Pack*>(dst + lane * VEC) = in[g];
      continue;
    }
    float x[VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      x[i] = __bfloat162float(in[g].v[i]);
      ss += x[i] * x[i];
    }
    if (p.has_norm) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
      for (int i = 0; i < VEC; ++i) x[i] = bf16_round(x[i] * inv * (kind == 0 ? qw[i] : kw[i]));
    }
    Pack out;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float partner = __shfl_xor_sync(0xFFFFFFFFu, x[i], half_lanes);
      out.v[i] = __float2bfloat16(rotated ? x[i] * cs[i] + partner * sn[i] : x[i]);
    }
    bf16* dst = kind == 0 ? p.q_out + ((long long)t * p.hq + h) * D : p.kv + (((page * 2 + 0) * p.page_size + off) * p.hkv + (h - p.hq)) * D;
    *reinterpret_cast<Pack*>(dst + lane * VEC) = out;
    if (kind == 0 && p.gated) {
      bf16* gdst = p.gate_out + ((long long)t * p.hq + h) * D;
      *reinterpret_cast<Pack*>(gdst + lane * VEC) = *reinterpret_cast<const Pack*>(src_of(h) + D + lane * VEC);
    }
  }
}

}  // namespace

extern "C" int pg_gather_rows(const void* table, const void* ids, void* out, int rows, int width, long long table_rows, void* status,
                              cudaStream_t stream) {
  PG_REQUIRE(width % 8 == 0, "gather_rows: width %d must be a multiple of 8", width);
  if (rows == 0) return PG_OK;
  PG_CUDA(launch_pdl(gather_rows_kernel, dim3(rows), dim3(128), (size_t)(0), stream, (const bf16*)table, (const int*)ids, (bf16*)out, rows, width, table_rows, (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_gather_words(const void* src, const void* idx, void* dst, int n, int src_len, void* status, cudaStream_t stream) {
  if (n <= 0) return PG_OK;
  PG_CUDA(launch_pdl(gather_words_kernel, dim3((n + 127) / 128), dim3(128), (size_t)(0), stream, (const uint32_t*)src, (const int*)idx, (uint32_t*)dst, n, src_len, (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_rms_norm(const void* x, void* residual, const void* w, void* y, int rows, int width, float eps, int offset, int round_before,
                           long long ldx, long long ldr, long long ldy, cudaStream_t stream) {
  PG_REQUIRE(width % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0, "rms_norm: width/strides must be multiples of 8");
  if (rows == 0) return PG_OK;
  if (residual)
    PG_CUDA(launch_pdl(rms_norm_kernel<1>, dim3(rows), dim3(256), (size_t)(0), stream, (const bf16*)x, (bf16*)residual, (const bf16*)w, (bf16*)y, width, eps, offset, round_before, ldx, ldr, ldy));
  else
    PG_CUDA(launch_pdl(rms_norm_kernel<0>, dim3(rows), dim3(256), (size_t)(0), stream, (const bf16*)x, nullptr, (const bf16*)w, (bf16*)y, width, eps, offset, 0, ldx, 0, ldy));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_gated_rms_norm_act(const void* x, const void* gate, const void* w_f32, void* y, long long rows, int dim, float eps, int act, cudaStream_t stream) {
  PG_REQUIRE(act == 0 || act == 1, "gated_rms_norm: gate activation %d (0 = SiLU, 1 = sigmoid)", act);
  if (rows == 0) return PG_OK;
  PG_CUDA(launch_pdl(gated_rms_norm_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), (size_t)(0), stream, (const bf16*)x, (const bf16*)gate, (const float*)w_f32, (bf16*)y, rows, dim, eps, act));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_gated_rms_norm(const void* x, const void* gate, const void* w_f32, void* y, long long rows, int dim, float eps, cudaStream_t stream) {
  return pg_gated_rms_norm_act(x, gate, w_f32, y, rows, dim, eps, 0, stream);
}

extern "C" int pg_swiglu(const void* gate_up, void* out, int rows, int inter, long long ldin, long long ldout, int interleaved, cudaStream_t stream) {
  PG_REQUIRE(inter % 8 == 0 && ldin % 8 == 0 && ldout % 8 == 0, "swiglu: sizes must be multiples of 8");
  if (rows == 0) return PG_OK;
  long long total = (long long)rows * (inter / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  PG_CUDA(launch_pdl(swiglu_kernel, dim3(blocks), dim3(256), (size_t)(0), stream, (const bf16*)gate_up, (bf16*)out, rows, inter, ldin, ldout, interleaved));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_softcap(const void* x, void* y, long long n, float cap, cudaStream_t stream) {
  PG_REQUIRE(cap > 0.f, "softcap: the cap must be positive");
  if (n == 0) return PG_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  PG_CUDA(launch_pdl(softcap_kernel, dim3((int)blocks), dim3(256), (size_t)(0), stream, (const bf16*)x, (bf16*)y, n, cap));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_sigmoid_gate_mul(void* x, const void* gate, long long n, cudaStream_t stream) {
  if (n == 0) return PG_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  PG_CUDA(launch_pdl(sigmoid_gate_mul_kernel, dim3((int)blocks), dim3(256), (size_t)(0), stream, (bf16*)x, (const bf16*)gate, n));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_qk_norm_rope_append(const void* qkv, long long ld, const void* q_w, const void* k_w, const void* cos, const void* sin,
                                      const void* positions, const void* slots, void* q_out, void* gate_out, void* kv, int tokens, int hq, int hkv,
                                      int dim, int rot, int page_size, long long num_pages, int max_pos, int gated, int offset, float eps,
                                      int v_norm, void* status, cudaStream_t stream) {
  PG_REQUIRE(dim % 8 == 0 && (dim <= 256 || dim == 512) && rot <= dim && rot % 2 == 0, "qk_norm_rope: unsupported head_dim %d / rotary %d", dim, rot);
  if (tokens == 0) return PG_OK;
  RopeParams p;
  p.qkv = (const bf16*)qkv;
  p.ld = ld;
  p.q_w = (const bf16*)q_w;
  p.k_w = (const bf16*)k_w;
  p.cos = (const bf16*)cos;
  p.sin = (const bf16*)sin;
  p.positions = (const int*)positions;
  p.slots = (const int*)slots;
  p.q_out = (bf16*)q_out;
  p.gate_out = (bf16*)gate_out;
  p.kv = (bf16*)kv;
  p.tokens = tokens;
  p.hq = hq;
  p.hkv = hkv;
  p.dim = dim;
  p.rot = rot;
  p.page_size = page_size;
  p.max_pos = max_pos;
  p.gated = gated;
  p.offset = offset;
  p.has_norm = q_w != nullptr;
  p.v_norm = v_norm;
  p.num_slots = num_pages * page_size;
  p.eps = eps;
  p.status = (uint32_t*)status;
  long long units = (long long)tokens * (hq + 2 * hkv);
  const int vec = dim / 32, half_lanes = (dim == 64 || dim == 128 || dim == 256 || dim == 512) && rot >= 2 * vec && (rot / 2) % vec == 0 ? rot / 2 / vec : 0;
  const bool vec_ok = half_lanes > 0 && (half_lanes & (half_lanes - 1)) == 0 && ld % (dim == 512 ? 16 : 8) == 0 && ((uintptr_t)qkv & (dim == 512 ? 31 : 15)) == 0;
  PG_REQUIRE(dim <= 256 || vec_ok, "qk_norm_rope: head dim 512 needs a rotary width whose half is a power-of-two multiple of 16 and 32-byte aligned rows");
  if (vec_ok) {
    const long long vunits = (long long)tokens * ((hq + 2 * hkv + ROPE_G - 1) / ROPE_G);
    const dim3 grid((unsigned)((vunits + 3) / 4));
    if (dim == 64) PG_CUDA(launch_pdl(qk_norm_rope_append_vec_kernel<2>, grid, dim3(128), (size_t)(0), stream, p));
    else if (dim == 128) PG_CUDA(launch_pdl(qk_norm_rope_append_vec_kernel<4>, grid, dim3(128), (size_t)(0), stream, p));
    else if (dim == 256) PG_CUDA(launch_pdl(qk_norm_rope_append_vec_kernel<8>, grid, dim3(128), (size_t)(0), stream, p));
    else PG_CUDA(launch_pdl(qk_norm_rope_append_vec_kernel<16>, grid, dim3(128), (size_t)(0), stream, p));
    PG_LAUNCH_CHECK();
    return PG_OK;
  }
  PG_CUDA(launch_pdl(qk_norm_rope_append_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), (size_t)(0), stream, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}


// ---------------------------------------------------------------------------------
// Load-time repack of compressed-tensors INT4 words: nibble j of the output word holds element
// (0, 2, 4, 6, 1, 3, 5, 7)[j] of the input word, so that the grouped GEMM gets two consecutive elements as one
// bf16 pair from a shift and a mask.  One 16-byte vector (32 weights) per thread.
// ---------------------------------------------------------------------------------
namespace {
__device__ __forceinline__ uint32_t pair_nibbles(uint32_t w) {
  // even elements to the low half, odd elements to the high half, order kept inside each half
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= ((w >> (8 * i)) & 0xFu) << (4 * i);
    hi |= ((w >> (8 * i + 4)) & 0xFu) << (4 * i);
  }
  return lo | (hi << 16);
}
__global__ void __launch_bounds__(256) repack_int4_pairs_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long vecs, const uint32_t* __restrict__ tail_in,
                                                                uint32_t* __restrict__ tail_out, int tail) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < vecs) {
    const uint4 v = in[i];
    out[i] = make_uint4(pair_nibbles(v.x), pair_nibbles(v.y), pair_nibbles(v.z), pair_nibbles(v.w));
  }
  if (i < tail) tail_out[i] = pair_nibbles(tail_in[i]);
}
}  // namespace

extern "C" int pg_repack_int4_pairs(const void* in, void* out, long long words, cudaStream_t stream) {
  if (words == 0) return PG_OK;
  PG_REQUIRE((((uintptr_t)in | (uintptr_t)out) & 15) == 0, "repack_int4_pairs: buffers must be 16-byte aligned");
  const long long vecs = words / 4;
  const int tail = (int)(words - vecs * 4);
  const long long threads = vecs > tail ? vecs : tail;
  repack_int4_pairs_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const uint4*)in, (uint4*)out, vecs, (const uint32_t*)in + vecs * 4,
                                                                                 (uint32_t*)out + vecs * 4, tail);
  PG_LAUNCH_CHECK();
  return PG_OK;
}
