// Grouped (per-expert) block-scaled FP8 GEMM on tcgen05 kind::f8f6f4 for mixture-of-experts layers.
//
//   Y[r, :] = dequant(Xq[r, :]) . dequant(Wq[e(r)])^T      rows r sorted by expert, expert e owns rows
//                                                          [offsets[e], offsets[e + 1])
//
//   Wq  e4m3 [E, M, K] with one f32 scale per 128 x 128 block, [E, M / 128, K / 128]
//   Xq  e4m3 [rows, K] with one f32 scale per row and 128-wide k group, stored [K / 128, ld]
//
// The activations are quantised per token group (pg_quant_fp8_1x128) instead of the weights being widened to bf16
// in shared memory: both operands reach the tensor core as e4m3 by TMA, at one byte per weight and four MMAs of
// K = 32 per 128-byte row.  As in the dense FP8 GEMM every k group goes into a fresh TMEM accumulator (two, ping-pong)
// and four warps read it back, multiply by scale_w * scale_x and add it into f32 registers while the tensor core
// multiplies the next group.  Work items (expert, weight-row tile, token tile) are derived on the device from
// `offsets`, so the launch shape does not depend on the routing and the kernel can sit inside a captured graph.
//
// Reference parity: pegainfer-kernels/csrc/glm52/glm52_deepgemm_grouped_sm100.cu (DeepGEMM masked grouped FP8 GEMM,
// cluster of two with multicast on A; here one CTA per item and no multicast), glm52_moe_quant.cu.
#include "common.cuh"

#include <cuda.h>

#include <mutex>

namespace {

constexpr int BM = 128, BKB = 128, MAX_STAGES = 6, MAX_EXPERTS = 512;
constexpr int A_BYTES = BM * BKB;

struct MoeFp8Params {
  const float* w_scale;  // [E, m_tiles, kgroups]
  const float* x_scale;  // [kgroups, ldxs]
  long long ldxs;
  bf16* y;
  long long ldy;
  const int* offsets;  // [E + 1]
  int M, E, kgroups, m_tiles, stages, kg_cap;
  uint32_t* status;
  // expert-parallel return path (as in the bf16 grouped kernel): output row r goes to rank (scatter_src[r] / cap), slot
  // (scatter_src[r] % cap) of that rank's combine buffer (row stride ldy); the tail raises the "returned" epoch
  const int* scatter_src;
  bf16* peer_out[8];
  uint32_t* peer_flags[8];
  int cap, rank, world, site;
};

__host__ __device__ constexpr uint32_t idesc_e4m3(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Item {
  int e, m_tile, row0, rows;
};
struct Cursor {
  int e = 0, base = 0;
};
// Items are ordered expert-major; s_tiles[e] = items of expert e.
template <int BN>
__device__ __forceinline__ bool locate(const MoeFp8Params& p, const int* s_tiles, int item, Cursor& c, Item& out) {
  while (c.e < p.E && item >= c.base + s_tiles[c.e]) {
    c.base += s_tiles[c.e];
    ++c.e;
  }
  if (c.e >= p.E) return false;
  const int local = item - c.base;
  const int n_tiles = s_tiles[c.e] / p.m_tiles;
  out.e = c.e;
  out.m_tile = local / n_tiles;
  const int n_tile = local - out.m_tile * n_tiles;
  const int r0 = p.offsets[c.e], r1 = p.offsets[c.e + 1];
  out.row0 = r0 + n_tile * BN;
  out.rows = min(BN, r1 - out.row0);
  return true;
}

template <int BN>
__global__ void __launch_bounds__(192) moe_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const MoeFp8Params p) {
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
  int* s_total = reinterpret_cast<int*>(tmem_slot + 2);
  float* s_ws = reinterpret_cast<float*>(tmem_slot + 4);  // [kg_cap] weight-block scales of the current item
  float* s_xs = s_ws + p.kg_cap;                           // [kgroups][BN] activation scales of the current item
  int* s_tiles = reinterpret_cast<int*>(s_xs + p.kg_cap * BN);
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
  PG_PDL_ENTRY();
  uint32_t ep_epoch = 0;
  if (p.scatter_src != nullptr) ep_epoch = *((volatile uint32_t*)(p.peer_flags[p.rank] + p.site * 32 + 16));
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_tiles[e] = p.m_tiles * ((p.offsets[e + 1] - p.offsets[e] + BN - 1) / BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int e = 0; e < p.E; ++e) tot += s_tiles[e];
    *s_total = tot;
  }
  __syncthreads();
  const uint32_t tmem_base = *tmem_slot;
  const int total = *s_total;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      long long n = 0;  // k groups loaded so far by this CTA
      Cursor cur;
      Item it;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        if (!locate<BN>(p, s_tiles, item, cur, it)) break;
        for (int kg = 0; kg < p.kgroups; ++kg, ++n) {
          if (n >= p.stages && !mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], (uint32_t)stage_bytes);
          uint8_t* st = tiles + stage * stage_bytes;
          tma_load_3d(st, &tm_w, &full[stage], kg * BKB, it.m_tile * BM, it.e, pol_w);
          tma_load_2d(st + A_BYTES, &tm_x, &full[stage], kg * BKB, it.row0, pol_x);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_e4m3(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      long long g = 0;  // k groups multiplied so far by this CTA: accumulator g & 1
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        for (int kg = 0; kg < p.kgroups; ++kg, ++g) {
          const int acc = (int)(g & 1);
          if (g >= 2 && !mbar_wait(&tempty[acc], (uint32_t)(((g >> 1) - 1) & 1), abort_flag)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty[stage]);
          umma_commit(&tfull[acc]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // read-back warps: warp w owns TMEM lanes 32 * (w % 4) ..; one weight row per thread
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int et = threadIdx.x - 64;  // 0..127
    long long g = 0;
    Cursor cur;
    Item it;
    bool ok = true;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      if (!locate<BN>(p, s_tiles, item, cur, it)) break;
      // the item's scales go to shared memory once (see the dense kernel)
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous item's scales are no longer read
      for (int i = et; i < p.kgroups; i += 128) s_ws[i] = p.w_scale[((long long)it.e * p.m_tiles + it.m_tile) * p.kgroups + i];
      for (int i = et; i < p.kgroups * BN; i += 128) {
        const int kg = i / BN, j = i % BN;
        s_xs[i] = j < it.rows ? p.x_scale[(long long)kg * p.ldxs + it.row0 + j] : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kg = 0; kg < p.kgroups; ++kg, ++g) {
        const int buf = (int)(g & 1);
        const float sw = s_ws[kg];
        const float4* sx = reinterpret_cast<const float4*>(s_xs + kg * BN);
        ok = mbar_wait(&tfull[buf], (uint32_t)((g >> 1) & 1), abort_flag);
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
      if (!ok) break;
      const int m = it.m_tile * BM + r;
      if (m < p.M) {
        if (p.scatter_src == nullptr) {
#pragma unroll
          for (int j = 0; j < BN; ++j)
            if (j < it.rows) p.y[(long long)(it.row0 + j) * p.ldy + m] = __float2bfloat16(acc[j]);
        } else {
#pragma unroll
          for (int j = 0; j < BN; ++j) {
            if (j < it.rows) {
              const int idx = p.scatter_src[it.row0 + j];
              const int dst_rank = idx / p.cap, slot = idx - dst_rank * p.cap;
              p.peer_out[dst_rank][(size_t)slot * p.ldy + m] = __float2bfloat16(acc[j]);
            }
          }
        }
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
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (32u << 8));
  if (p.scatter_src != nullptr && threadIdx.x == 0) {
    // every output row of this CTA is on its way to its source rank (the barrier above orders the other threads'
    // stores before this fence): the last CTA of this GPU raises the "returned" epoch on all ranks
    uint32_t* myflags = p.peer_flags[p.rank] + p.site * 32;
    __threadfence_system();
    const uint32_t old = atomicAdd(&myflags[17], 1u);
    if (old == gridDim.x - 1) {
      myflags[17] = 0u;
      for (int q = 0; q < p.world; ++q) st_release_sys(p.peer_flags[q] + p.site * 32 + 8 + p.rank, ep_epoch + 1u);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

template <int BN>
int launch(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const MoeFp8Params& p, int sms, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)p.stages * (A_BYTES + BN * BKB) + (2 * MAX_STAGES + 4) * 8 + 64 + (size_t)p.kg_cap * (BN + 1) * 4 + (size_t)MAX_EXPERTS * 4;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(moe_gemm_fp8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(moe_gemm_fp8_kernel<BN>, dim3((unsigned)(2 * sms)), dim3(192), smem, stream, tm_w, tm_x, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

}  // namespace

// xq [rows, K] e4m3 (row stride K), x_scale [K / 128, ldxs] f32, wq [E, M, K] e4m3, w_scale [E, M / 128, K / 128] f32,
// y [rows, M] bf16, offsets [E + 1] int32 (device).  `bn`: token tile, 16, 32 or 64.
static int moe_fp8_impl(const void* xq, long long rows, const void* x_scale, long long ldxs, const void* wq, const void* w_scale, void* y, long long ldy, const void* offsets,
                        int E, int M, int K, int bn, void* status, const void* scatter_src, void* const* peer_out, void* const* peer_flags, int cap, int rank, int world,
                        int site, cudaStream_t stream) {
  PG_REQUIRE(K % 128 == 0 && M % 128 == 0, "fp8 grouped gemm: K %d and M %d must be multiples of the 128 x 128 scale block", K, M);
  PG_REQUIRE(E >= 1 && E <= MAX_EXPERTS, "fp8 grouped gemm: %d experts (at most %d)", E, MAX_EXPERTS);
  PG_REQUIRE(bn == 16 || bn == 32 || bn == 64, "fp8 grouped gemm: token tile %d", bn);
  if (rows == 0 && scatter_src == nullptr) return PG_OK;
  PG_REQUIRE(rows > 0, "fp8 grouped gemm: the return path needs a non-empty row buffer");
  EncodeTiledFn enc = get_encode();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE((((uintptr_t)xq | (uintptr_t)wq) & 15) == 0, "TMA base addresses must be 16-byte aligned");
  CUtensorMap tm_w, tm_x;
  {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)M * (cuuint64_t)K};
    cuuint32_t box[3] = {128u, (cuuint32_t)BM, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(wq), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (weights) failed with code %d", (int)r);
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128u, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(xq), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (activations) failed with code %d", (int)r);
  }
  MoeFp8Params p;
  p.w_scale = (const float*)w_scale;
  p.x_scale = (const float*)x_scale;
  p.ldxs = ldxs;
  p.y = (bf16*)y;
  p.ldy = ldy;
  p.offsets = (const int*)offsets;
  p.M = M;
  p.E = E;
  p.kgroups = K / 128;
  p.m_tiles = M / BM;
  p.kg_cap = (p.kgroups + 4) & ~3;
  p.stages = 4;
  p.status = (uint32_t*)status;
  p.scatter_src = (const int*)scatter_src;
  p.cap = p.rank = p.world = p.site = 0;
  if (scatter_src) {
    for (int q = 0; q < world; ++q) {
      p.peer_out[q] = (bf16*)peer_out[q];
      p.peer_flags[q] = (uint32_t*)peer_flags[q];
    }
    p.cap = cap;
    p.rank = rank;
    p.world = world;
    p.site = site;
  }
  int dev = 0, sms = 148;
  PG_CUDA(cudaGetDevice(&dev));
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (bn == 16) return launch<16>(tm_w, tm_x, p, sms, stream);
  if (bn == 32) return launch<32>(tm_w, tm_x, p, sms, stream);
  return launch<64>(tm_w, tm_x, p, sms, stream);
}

extern "C" int pg_moe_grouped_gemm_fp8(const void* xq, long long rows, const void* x_scale, long long ldxs, const void* wq, const void* w_scale, void* y, long long ldy,
                                       const void* offsets, int E, int M, int K, int bn, void* status, cudaStream_t stream) {
  return moe_fp8_impl(xq, rows, x_scale, ldxs, wq, w_scale, y, ldy, offsets, E, M, K, bn, status, nullptr, nullptr, nullptr, 0, 0, 1, 0, stream);
}

// Expert-parallel W2 on the FP8 tensor-core path: output rows are stored straight into their source ranks' combine
// buffers (row stride ldy) and the kernel's tail raises this rank's "returned" epoch.
extern "C" int pg_moe_grouped_gemm_fp8_return(const void* xq, long long rows, const void* x_scale, long long ldxs, const void* wq, const void* w_scale, long long ldy,
                                              const void* offsets, int E, int M, int K, int bn, void* status, const void* scatter_src, void* const* peer_out,
                                              void* const* peer_flags, int cap, int rank, int world, int site, cudaStream_t stream) {
  PG_REQUIRE(scatter_src != nullptr && world >= 1 && world <= 8, "fp8 grouped gemm return: needs the sorted-source table and 1..8 ranks");
  return moe_fp8_impl(xq, rows, x_scale, ldxs, wq, w_scale, nullptr, ldy, offsets, E, M, K, bn, status, scatter_src, peer_out, peer_flags, cap, rank, world, site, stream);
}
