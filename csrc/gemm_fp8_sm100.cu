// Block-scaled FP8 GEMM for sm_100a: Y[T, M] = dequant(Xq)[T, K] . dequant(Wq)[M, K]^T on tcgen05 (kind::f8f6f4).
//
//   Wq  e4m3 [M, K], one f32 scale per 128 x 128 block  (checkpoint layout: weight + weight_scale_inv)
//   Xq  e4m3 [T, K], one f32 scale per token and 128-wide k group, stored [K / 128, T] so that a tile reads
//       its tokens' scales of one k group as one contiguous run (pg_quant_fp8_1x128 writes this layout)
//
// Both operands are staged by TMA as K-major tiles with the 128-byte swizzle: one 128-byte row is one k group
// of 128 e4m3 values, i.e. four MMAs of K = 32.  The scales differ from k group to k group, so a k group's
// product may not be added into the running sum inside the tensor core: every k group is multiplied into a
// fresh TMEM accumulator (two of them, ping-pong), and four warps read it back (tcgen05.ld), multiply by
// scale_w * scale_x and add it into f32 registers while the tensor core works on the next k group.  A decode
// GEMM is bound by the weight stream (half the bytes of bf16), which leaves several hundred cycles per k group
// for that read-back.  Narrow token tiles split K over grid.z; the partial sums go to a workspace and a small
// kernel adds them in split order (deterministic).
//
// Reference parity: pegainfer-kernels/csrc/glm52/{glm52_fp8_gemm.cu (CUTLASS groupwise-scaled FP8 GEMM),
// glm52_moe_quant.cu (per-token-group FP8 quantisation)}, pegainfer-glm52/src/fp8.rs (128 x 128 weight blocks).
#include "common.cuh"

#include <cuda.h>
#include <cuda_fp8.h>

#include <mutex>

namespace {

constexpr int BM = 128;       // weight rows per tile (UMMA M)
constexpr int BKB = 128;      // bytes = e4m3 values per k group
constexpr int MAX_STAGES = 8;
constexpr int A_BYTES = BM * BKB;

struct Fp8Params {
  const float* w_scale;  // [m_tiles, kgroups]
  const float* x_scale;  // [kgroups, ldxs]
  long long ldxs;
  bf16* y;
  long long ldy;
  float* ws;  // [splits, T, M] f32 when splits > 1
  int M, T, kgroups, bn, stages, splits, m_tiles, n_tiles, kg_cap;
  uint32_t* status;
};

// kind::f8f6f4, e4m3 x e4m3 -> f32, both operands K-major
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int BN>
__global__ void __launch_bounds__(192) gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  constexpr int stage_bytes = A_BYTES + BN * BKB;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_ws = reinterpret_cast<float*>(tmem_slot + 4);  // [k groups of this CTA] weight-block scales
  float* s_xs = s_ws + p.kg_cap;                           // [k groups of this CTA][BN] activation scales (0 past T)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  PG_PDL_ENTRY();

  const int m_tile = blockIdx.x, n_tile = blockIdx.y, split = blockIdx.z;
  const int kg0 = (int)(((long long)p.kgroups * split) / p.splits);
  const int kg1 = (int)(((long long)p.kgroups * (split + 1)) / p.splits);

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      for (int kg = kg0; kg < kg1; ++kg) {
        if (kg - kg0 >= p.stages && !mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) break;
        mbar_expect_tx(&full[stage], (uint32_t)stage_bytes);
        uint8_t* st = tiles + stage * stage_bytes;
        tma_load_2d(st, &tm_w, &full[stage], kg * BKB, m_tile * BM, pol_w);
        tma_load_2d(st + A_BYTES, &tm_x, &full[stage], kg * BKB, n_tile * BN, pol_x);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      for (int kg = kg0; kg < kg1; ++kg) {
        const int i = kg - kg0, acc = i & 1;
        // the read-back warps have drained this accumulator's previous k group
        if (i >= 2 && !mbar_wait(&tempty[acc], (uint32_t)(((i >> 1) - 1) & 1), abort_flag)) break;
        if (!mbar_wait(&full[stage], phase, abort_flag)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
        const uint32_t b_addr = a_addr + A_BYTES;
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8_ss(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, k > 0 ? 1u : 0u);
        umma_commit(&empty[stage]);
        umma_commit(&tfull[acc]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // read-back warps: warp w owns TMEM lanes 32 * (w % 4) ..; one weight row per thread
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int m = m_tile * BM + r;
    const int n0 = n_tile * BN;
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    // this CTA's scales go to shared memory once: read per k group from global memory they would put a memory
    // latency and BN loads per thread on the critical path of every k group
    const int et = threadIdx.x - 64;  // 0..127
    for (int i = et; i < kg1 - kg0; i += 128) s_ws[i] = p.w_scale[(long long)m_tile * p.kgroups + kg0 + i];
    for (int i = et; i < (kg1 - kg0) * BN; i += 128) {
      const int g = i / BN, j = i % BN;
      s_xs[i] = (n0 + j < p.T) ? p.x_scale[(long long)(kg0 + g) * p.ldxs + n0 + j] : 0.f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    bool ok = true;
    for (int kg = kg0; kg < kg1 && ok; ++kg) {
      const int i = kg - kg0, buf = i & 1;
      const float sw = s_ws[i];
      const float4* sx = reinterpret_cast<const float4*>(s_xs + i * BN);
      ok = mbar_wait(&tfull[buf], (uint32_t)((i >> 1) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float4 s4 = sx[(c >> 2) + q4];
          acc[c + q4 * 4 + 0] = fmaf(__uint_as_float(v[q4 * 4 + 0]), sw * s4.x, acc[c + q4 * 4 + 0]);
          acc[c + q4 * 4 + 1] = fmaf(__uint_as_float(v[q4 * 4 + 1]), sw * s4.y, acc[c + q4 * 4 + 1]);
          acc[c + q4 * 4 + 2] = fmaf(__uint_as_float(v[q4 * 4 + 2]), sw * s4.z, acc[c + q4 * 4 + 2]);
          acc[c + q4 * 4 + 3] = fmaf(__uint_as_float(v[q4 * 4 + 3]), sw * s4.w, acc[c + q4 * 4 + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    if (ok && m < p.M) {
      if (p.splits == 1) {
#pragma unroll
        for (int j = 0; j < BN; ++j)
          if (n0 + j < p.T) p.y[(long long)(n0 + j) * p.ldy + m] = __float2bfloat16(acc[j]);
      } else {
        float* wsp = p.ws + ((long long)split * p.T) * p.M;
#pragma unroll
        for (int j = 0; j < BN; ++j)
          if (n0 + j < p.T) wsp[(long long)(n0 + j) * p.M + m] = acc[j];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (31u << 8));
}

__global__ void __launch_bounds__(256) fp8_splitk_sum_kernel(const float* __restrict__ ws, int splits, long long tm, int M, bf16* __restrict__ y, long long ldy) {
  PG_PDL_ENTRY();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= tm) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += ws[(long long)k * tm + i];
  y[(i / M) * ldy + (i % M)] = __float2bfloat16(s);
}

// one warp per (token, k group): amax -> scale = amax / 448, values rounded to e4m3
__global__ void __launch_bounds__(128) quant_fp8_1x128_kernel(const bf16* __restrict__ x, long long ldx, int T, int kgroups, uint8_t* __restrict__ xq, long long ldq,
                                                               float* __restrict__ scale, long long lds) {
  PG_PDL_ENTRY();
  const long long u = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (u >= (long long)T * kgroups) return;
  const int t = (int)(u / kgroups), g = (int)(u % kgroups), lane = threadIdx.x & 31;
  const bf16* src = x + (long long)t * ldx + g * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const bf162 a = *reinterpret_cast<const bf162*>(&raw.x), b = *reinterpret_cast<const bf162*>(&raw.y);
  float v[4] = {__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y)};
  const float amax = fmaxf(warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])))), 1e-10f);
  const float s = amax / 448.f, inv = 448.f / amax;
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) out |= (uint32_t)__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * i);
  *reinterpret_cast<uint32_t*>(xq + (long long)t * ldq + g * 128 + lane * 4) = out;
  if (lane == 0) scale[(long long)g * lds + t] = s;
}

// SwiGLU and the quantiser in one pass: gu [T, 2 K] bf16 (gate half first) -> e4m3 of round_bf16(round_bf16(silu(gate)) * up)
// with the same per-token, per-k-group scales; bit-identical to the swiglu kernel followed by the quantiser.
__global__ void __launch_bounds__(128) swiglu_quant_fp8_1x128_kernel(const bf16* __restrict__ gu, long long ldx, int T, int kgroups, uint8_t* __restrict__ xq, long long ldq,
                                                                      float* __restrict__ scale, long long lds) {
  PG_PDL_ENTRY();
  const long long u = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (u >= (long long)T * kgroups) return;
  const int t = (int)(u / kgroups), g = (int)(u % kgroups), lane = threadIdx.x & 31;
  const bf16* src = gu + (long long)t * ldx + g * 128 + lane * 4;
  const uint2 rg = *reinterpret_cast<const uint2*>(src), ru = *reinterpret_cast<const uint2*>(src + (long long)kgroups * 128);
  const bf16* pg = reinterpret_cast<const bf16*>(&rg);
  const bf16* pu = reinterpret_cast<const bf16*>(&ru);
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float gf = __bfloat162float(pg[i]);
    const float sg = __bfloat162float(__float2bfloat16(gf / (1.f + __expf(-gf))));
    v[i] = __bfloat162float(__float2bfloat16(sg * __bfloat162float(pu[i])));
  }
  const float amax = fmaxf(warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])))), 1e-10f);
  const float s = amax / 448.f, inv = 448.f / amax;
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) out |= (uint32_t)__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * i);
  *reinterpret_cast<uint32_t*>(xq + (long long)t * ldq + g * 128 + lane * 4) = out;
  if (lane == 0) scale[(long long)g * lds + t] = s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fp8() {
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

// Row-major [rows, cols] byte matrix with row stride ld bytes; box = [box_rows x 128 bytes], 128-byte swizzle.
int make_tmap_u8_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fp8();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0 && ld % 16 == 0, "TMA base address and row stride must be multiples of 16 bytes");
  PG_REQUIRE(box_rows >= 1 && box_rows <= 256, "unsupported TMA box of %d rows", box_rows);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}

template <int BN>
int launch_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const Fp8Params& p, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)p.stages * (A_BYTES + BN * BKB) + (2 * MAX_STAGES + 4) * 8 + 64 + (size_t)p.kg_cap * (BN + 1) * 4;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(gemm_fp8_block_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(gemm_fp8_block_kernel<BN>, dim3((unsigned)p.m_tiles, (unsigned)p.n_tiles, (unsigned)p.splits), dim3(192), smem, stream, tm_w, tm_x, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

}  // namespace

extern "C" long long pg_gemm_fp8_ws_bytes(int T, int M) { return 16ll * T * M * 4; }

// Y[T, M] (bf16, row stride ldy) = (Xq * x_scale) . (Wq * w_scale)^T.  ``ws``: pg_gemm_fp8_ws_bytes(T, M) bytes.
extern "C" int pg_gemm_fp8_block(const void* xq, long long ldx, const void* x_scale, long long ldxs, const void* wq, long long ldw, const void* w_scale, void* y,
                                 long long ldy, int T, int M, int K, void* ws, long long ws_bytes, void* status, cudaStream_t stream) {
  PG_REQUIRE(K % 128 == 0 && M % 128 == 0, "fp8 gemm: K %d and M %d must be multiples of the 128 x 128 scale block", K, M);
  if (T == 0) return PG_OK;
  Fp8Params p;
  p.w_scale = (const float*)w_scale;
  p.x_scale = (const float*)x_scale;
  p.ldxs = ldxs;
  p.y = (bf16*)y;
  p.ldy = ldy;
  p.ws = (float*)ws;
  p.M = M;
  p.T = T;
  p.kgroups = K / 128;
  p.bn = T <= 16 ? 16 : T <= 32 ? 32 : 64;
  p.m_tiles = M / BM;
  p.n_tiles = ceil_div(T, p.bn);
  p.status = (uint32_t*)status;
  int dev = 0, sms = 148;
  PG_CUDA(cudaGetDevice(&dev));
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // split K until the grid covers the SMs about twice (the weight stream is what a narrow GEMM waits for)
  int splits = 1;
  while (splits < 16 && p.m_tiles * p.n_tiles * splits * 2 <= 2 * sms && p.kgroups / (splits * 2) >= 4) splits *= 2;
  if ((long long)splits * T * M * 4 > ws_bytes) splits = 1;
  p.splits = splits;
  const int per = ceil_div(p.kgroups, splits);
  p.kg_cap = (per + 4) & ~3;  // k groups of one CTA, rounded for the float4 reads of the staged scales
  // four stages leave room for two CTAs per SM (a grid of 150 - 296 CTAs then runs as one wave)
  p.stages = min(4, max(2, per));
  CUtensorMap tm_w, tm_x;
  int rc = make_tmap_u8_2d(&tm_w, wq, M, K, ldw, BM);
  if (rc != PG_OK) return rc;
  rc = make_tmap_u8_2d(&tm_x, xq, T, K, ldx, p.bn);
  if (rc != PG_OK) return rc;
  if (p.bn == 16) rc = launch_fp8<16>(tm_w, tm_x, p, stream);
  else if (p.bn == 32) rc = launch_fp8<32>(tm_w, tm_x, p, stream);
  else rc = launch_fp8<64>(tm_w, tm_x, p, stream);
  if (rc != PG_OK) return rc;
  if (splits > 1) {
    const long long tm = (long long)T * M;
    PG_CUDA(launch_pdl(fp8_splitk_sum_kernel, dim3((unsigned)((tm + 255) / 256)), dim3(256), (size_t)0, stream, (const float*)ws, splits, tm, M, (bf16*)y, ldy));
    PG_LAUNCH_CHECK();
  }
  return PG_OK;
}

// x [T, K] bf16 -> xq [T, K] e4m3 + scale [K / 128, lds] f32 (scale of token t and group g at [g, t]).
extern "C" int pg_quant_fp8_1x128(const void* x, long long ldx, int T, int K, void* xq, long long ldq, void* scale, long long lds, cudaStream_t stream) {
  PG_REQUIRE(K % 128 == 0 && ldx % 4 == 0 && ldq % 4 == 0, "fp8 quant: K %d must be a multiple of 128", K);
  const long long units = (long long)T * (K / 128);
  if (units == 0) return PG_OK;
  PG_CUDA(launch_pdl(quant_fp8_1x128_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), (size_t)0, stream, (const bf16*)x, ldx, T, K / 128, (uint8_t*)xq, ldq,
                     (float*)scale, lds));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// gu [T, 2 K] bf16 (gate half first) -> xq [T, K] e4m3 of SwiGLU(gu) + scale [K / 128, lds] f32.
extern "C" int pg_swiglu_quant_fp8_1x128(const void* gu, long long ldx, int T, int K, void* xq, long long ldq, void* scale, long long lds, cudaStream_t stream) {
  PG_REQUIRE(K % 128 == 0 && ldx % 4 == 0 && ldq % 4 == 0, "fp8 swiglu quant: K %d must be a multiple of 128", K);
  const long long units = (long long)T * (K / 128);
  if (units == 0) return PG_OK;
  PG_CUDA(launch_pdl(swiglu_quant_fp8_1x128_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), (size_t)0, stream, (const bf16*)gu, ldx, T, K / 128, (uint8_t*)xq, ldq,
                     (float*)scale, lds));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
