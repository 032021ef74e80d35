// Grouped (per-expert) GEMM on tcgen05 for mixture-of-experts layers.
//
//   Y[r, :] = X[r, :] * W[e(r)]^T      rows r sorted by expert, expert e owns rows
//                                      [offsets[e], offsets[e+1])
//
// Same operand roles as the dense GEMM: 128 weight rows of one expert are the UMMA A
// operand, a tile of that expert's token rows is the B operand, so an expert with two
// tokens still runs full-width MMAs and the kernel streams each expert's weights once
// (the MoE-GEMV regime of decode).  Work items (expert, weight-row tile, token tile) are
// derived on the device from `offsets`, so the launch shape does not depend on the
// routing and the kernel can sit inside a captured graph.
//
// Weight formats:
//   bf16   W [E, M, K]: TMA straight into the swizzled A tile.
//   int4   W packed [E, M, K/8] int32 (offset-binary nibbles, pair-interleaved inside each word:
//          bits 0-15 hold elements 0,2,4,6 and bits 16-31 elements 1,3,5,7 of the word's eight) with
//          bf16 scales [E, M, K/32]: TMA brings the packed tile (4 KB per 128x64) into a
//          raw buffer, the dequantisation warps (four groups of two, each group taking every
//          fourth k-block) expand it to bf16 ((nibble - 8) * scale,
//          one rounding) directly into the 128-byte-swizzled A tile and hand it to the MMA
//          warp through an mbarrier; HBM traffic stays at 4.5 bits per weight.
//   fp8    W e4m3 [E, M, K] with f32 scale_inv [E, ceil(M/128), ceil(K/128)] (block-scaled
//          checkpoints): TMA brings the raw 8 KB tile, the same warps convert e4m3 ->
//          f32 (exact), multiply by the block's scale_inv and round once to bf16 into the
//          swizzled A tile; HBM traffic is one byte per weight.
//
// warp 0 TMA producer | warp 1 MMA issuer + TMEM owner | warps 2-5 epilogue | warps 6-13 dequant (int4 / fp8)
//
// Takes the place of the reference's Marlin W4A16 MoE kernel
// (pegainfer-kernels/csrc/kimi_k2/kimi_marlin_wna16.cu:241-340, vllm_marlin/**) and its
// per-expert dense GEMM loop (pegainfer-deepseek-v2-lite/src/runtime/moe.rs).
#include <string.h>

#include <mutex>

#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int RAW_BYTES = BM * BK / 2;  // packed int4 tile
constexpr int RAW_BYTES_FP8 = BM * BK;  // fp8 tile
constexpr int MAX_STAGES = 10;
constexpr int MAX_EXPERTS = 512;

struct MoeGemmParams {
  bf16* y;
  long long ldy;
  int M, K, E;
  int bn, stages, kblocks, m_tiles;
  uint32_t tmem_cols;
  int quant;           // 0 bf16, 1 int4 group-32, 2 fp8 e4m3 with 128x128 block scales
  const void* scales;  // int4: bf16 [E, M, K/32]; fp8: f32 scale_inv [E, ceil(M/128), ceil(K/128)]
  const int* offsets;  // [E+1]
  uint32_t* status;
  // expert-parallel return path: output row r goes to rank (scatter_src[r] / cap), slot
  // (scatter_src[r] % cap) of that rank's combine buffer; the tail raises the "returned" epoch
  const int* scatter_src;
  bf16* peer_out[8];
  uint32_t* peer_flags[8];
  int cap, rank, world, site;
};

struct Item {
  int e, m_tile, row0, rows;
};

// Items are ordered expert-major; `cum` holds the running item count of experts before `e`.
struct ItemCursor {
  int e = 0;
  int base = 0;
};

__device__ __forceinline__ bool locate(const MoeGemmParams& p, const int* s_tiles, int item, ItemCursor& c, Item& out) {
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
  out.row0 = r0 + n_tile * p.bn;
  out.rows = min(p.bn, r1 - out.row0);
  return true;
}

__device__ __forceinline__ bool named_bar_all(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(nthreads)
      : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(448, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const MoeGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_tiles[MAX_EXPERTS];
  __shared__ int s_total;
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  const int b_bytes = p.bn * 128;
  const int raw_bytes = p.quant == 1 ? RAW_BYTES : p.quant == 2 ? RAW_BYTES_FP8 : 0;
  const int stage_bytes = A_BYTES + b_bytes + raw_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* aready = empty + MAX_STAGES;
  uint64_t* tfull = aready + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&aready[s], 64);  // one dequant group
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
  // per-expert item counts (every CTA derives the same list from the routing offsets)
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const int n = p.offsets[e + 1] - p.offsets[e];
    s_tiles[e] = n > 0 ? p.m_tiles * ((n + p.bn - 1) / p.bn) : 0;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < p.E; ++e) t += s_tiles[e];
    s_total = t;
  }
  __syncthreads();
  const uint32_t tmem_base = *tmem_slot;
  const int total = s_total;
  uint32_t ep_epoch = 0;
  if (p.scatter_src != nullptr) ep_epoch = *((volatile uint32_t*)(p.peer_flags[p.rank] + p.site * 32 + 16));

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t last_phase[MAX_STAGES];
      bool used[MAX_STAGES];
#pragma unroll
      for (int s = 0; s < MAX_STAGES; ++s) {
        used[s] = false;
        last_phase[s] = 0;
      }
      ItemCursor cur;
      Item it;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        if (!locate(p, s_tiles, item, cur, it)) break;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* st = tiles + stage * stage_bytes;
          if (p.quant) {
            mbar_expect_tx(&full[stage], (uint32_t)(raw_bytes + b_bytes));
            tma_load_3d(st + A_BYTES + b_bytes, &tm_w, &full[stage], p.quant == 1 ? kb * (BK / 8) : kb * BK, it.m_tile * BM, it.e, pol_w);
          } else {
            mbar_expect_tx(&full[stage], (uint32_t)(A_BYTES + b_bytes));
            tma_load_3d(st, &tm_w, &full[stage], kb * BK, it.m_tile * BM, it.e, pol_w);
          }
          tma_load_2d(st + A_BYTES, &tm_x, &full[stage], kb * BK, it.row0, pol_x);
          used[stage] = true;
          last_phase[stage] = phase;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      for (int s = 0; s < p.stages; ++s) {
        if (!used[s]) continue;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&full[s], last_phase[s])) {
          if (globaltimer_ns() - t0 > PG_WAIT_LIMIT_NS) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(BM, (uint32_t)p.bn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          // quantised weights: a_ready implies the raw tile and X landed and the bf16 A tile is written
          if (!mbar_wait(p.quant ? &aready[stage] : &full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_ss(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < 6) {
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    ItemCursor cur;
    Item it;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      if (!locate(p, s_tiles, item, cur, it)) break;
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag);
      ok = named_bar_all(1, 128, ok);
      if (!ok) break;
      tc_fence_after();
      const int m = it.m_tile * BM + r;
      const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * p.bn);
      for (int c = 0; c < p.bn; c += 16) {
        if (c >= it.rows) break;  // uniform across the warp
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
        if (m < p.M) {
          if (p.scatter_src == nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < it.rows) p.y[(size_t)(it.row0 + c + j) * p.ldy + m] = __float2bfloat16(__uint_as_float(v[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < it.rows) {
                const int idx = p.scatter_src[it.row0 + c + j];
                const int dst_rank = idx / p.cap, slot = idx - dst_rank * p.cap;
                p.peer_out[dst_rank][(size_t)slot * p.ldy + m] = __float2bfloat16(__uint_as_float(v[j]));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else if (p.quant != 0) {
    // Dequantisation warps.  The chain of one k-block (raw tile landed -> expand -> write the
    // swizzled bf16 A tile -> proxy fence -> hand to the MMA warp) has a latency of several
    // hundred cycles that no single group of threads can hide, so the eight warps form four
    // groups of 64 threads and group g takes every fourth k-block (counted across work items):
    // four tiles are being expanded at any time.  A thread expands rows t and t + 64.  The stage
    // count is a multiple of 4 (host side), so group g only ever touches stages = g (mod 4).
    const int dq = threadIdx.x - 192;  // 0..255
    const int grp = dq >> 6, t = dq & 63;
    ItemCursor cur;
    Item it;
    long long kbg0 = 0;  // global index of this item's first k-block
    bool ok = true;
    const bool int4 = p.quant == 1;
    const int groups_per_row = p.K / 32;
    const int mb = (p.M + 127) / 128, kbk = (p.K + 127) / 128;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x, kbg0 += p.kblocks) {
      if (!locate(p, s_tiles, item, cur, it)) break;
      const int first = (int)(((long long)grp - kbg0) & 3);  // first k-block of this item that belongs to the group
      // scales of the group's next k-block are fetched one turn (four k-blocks) ahead
      const bf16* srow[2];
      bool live[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int m = it.m_tile * BM + t + 64 * h;
        live[h] = m < p.M;
        srow[h] = reinterpret_cast<const bf16*>(p.scales) + ((size_t)it.e * p.M + (live[h] ? m : 0)) * groups_per_row;
      }
      const float* frow = reinterpret_cast<const float*>(p.scales) + ((size_t)it.e * mb + it.m_tile) * kbk;
      const bf16 zero = __float2bfloat16(0.f);
      bf16 sc[2][2], nx[2][2];
      float fs = 0.f, fnx = 0.f;
      auto load_scales = [&](int kb, bf16 (&dst)[2][2], float& fdst) {
        if (kb >= p.kblocks) return;
        if (int4) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            dst[h][0] = (live[h] && kb * 2 < groups_per_row) ? srow[h][kb * 2] : zero;
            dst[h][1] = (live[h] && kb * 2 + 1 < groups_per_row) ? srow[h][kb * 2 + 1] : zero;
          }
        } else {
          fdst = frow[kb >> 1];
        }
      };
      load_scales(first, sc, fs);
      for (int kb = first; kb < p.kblocks && ok; kb += 4) {
        load_scales(kb + 4, nx, fnx);
        const long long kbg = kbg0 + kb;
        const int stage = (int)(kbg % p.stages);
        const uint32_t phase = (uint32_t)((kbg / p.stages) & 1);
        if (!mbar_wait(&full[stage], phase, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* st = tiles + stage * stage_bytes;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = t + 64 * h;
          uint8_t* a_row = st + r * 128;
          if (int4) {
            const uint4* raw = reinterpret_cast<const uint4*>(st + A_BYTES + b_bytes + r * 32);
            const bf162 bias = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const uint4 rw = raw[hf];
              const uint32_t words[4] = {rw.x, rw.y, rw.z, rw.w};
              const bf162 s2 = __halves2bfloat162(sc[h][hf], sc[h][hf]);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                // pair-interleaved nibbles: (w >> 4i) & 0x000F000F | 0x43004300 = bf16 pair (128 + e[2i], 128 + e[2i+1])
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint32_t tt = ((words[c] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
                  bf162 val = *reinterpret_cast<bf162*>(&tt);
                  val = __hmul2(__hsub2(val, bias), s2);
                  o[i] = *reinterpret_cast<uint32_t*>(&val);
                }
                const int ch = hf * 4 + c;
                *reinterpret_cast<uint4*>(a_row + ((ch ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          } else {
            // fp8 e4m3: exact in half, f32 * scale_inv of the 128x128 block, rounded once to bf16
            const uint4* raw = reinterpret_cast<const uint4*>(st + A_BYTES + b_bytes + r * 64);
#pragma unroll
            for (int half = 0; half < 4; ++half) {
              const uint4 v = raw[half];
              const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint32_t w = words[hh * 2 + (q >> 1)];
                  const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((w >> (16 * (q & 1))) & 0xFFFFu);
                  const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
                  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
                  const bf162 b2 = __floats2bfloat162_rn(f.x * fs, f.y * fs);
                  o[q] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                const int ch = half * 2 + hh;
                *reinterpret_cast<uint4*>(a_row + ((ch ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&aready[stage]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          sc[h][0] = nx[h][0];
          sc[h][1] = nx[h][1];
        }
        fs = fnx;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (5u << 8));
  if (p.scatter_src != nullptr && threadIdx.x == 0) {
    // every output row of this CTA is on its way to its source rank: the last CTA of this
    // GPU raises the "returned" epoch on all ranks
    uint32_t* myflags = p.peer_flags[p.rank] + p.site * 32;
    __threadfence_system();
    const uint32_t old = atomicAdd(&myflags[17], 1u);
    if (old == gridDim.x - 1) {
      myflags[17] = 0u;
      for (int q = 0; q < p.world; ++q) st_release_sys(p.peer_flags[q] + p.site * 32 + 8 + p.rank, ep_epoch + 1u);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn moe_get_encode() {
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

bool g_attr_set[64];
int g_sms[64], g_max_smem[64];
int g_static_smem = 0;
std::mutex g_mu;

}  // namespace

// x [rows, K] bf16 (rows sorted by expert), offsets [E+1] device int32, y [rows, M] bf16.
// w: bf16 [E, M, K] (quant 0); packed int32 [E, M, K/8] with scales bf16 [E, M, K/32] (quant 1);
// fp8 e4m3 [E, M, K] with f32 scale_inv [E, ceil(M/128), ceil(K/128)] (quant 2).
// `bn` is the token tile (multiple of 16, <= 256): pick it near the expected rows per expert.
static int moe_gemm_impl(const void* x, long long ldx, long long x_rows, const void* w, const void* scales, int quant, void* y, long long ldy,
                         const void* offsets, int E, int M, int K, int bn, void* status, const void* scatter_src, void* const* peer_out,
                         void* const* peer_flags, int cap, int rank, int world, int site, cudaStream_t stream) {
  PG_REQUIRE(E >= 1 && E <= MAX_EXPERTS, "moe gemm: %d experts not supported (<= %d)", E, MAX_EXPERTS);
  PG_REQUIRE(K % 64 == 0, "moe gemm: K=%d must be a multiple of 64", K);
  PG_REQUIRE(bn >= 16 && bn <= 256 && bn % 16 == 0, "moe gemm: token tile %d must be a multiple of 16 in [16, 256]", bn);
  PG_REQUIRE(status != nullptr, "moe gemm: a device status word is required");
  if (x_rows == 0 && scatter_src == nullptr) return PG_OK;
  EncodeTiledFn enc = moe_get_encode();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_attr_set[dev & 63]) {
      PG_CUDA(cudaDeviceGetAttribute(&g_sms[dev & 63], cudaDevAttrMultiProcessorCount, dev));
      PG_CUDA(cudaDeviceGetAttribute(&g_max_smem[dev & 63], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      cudaFuncAttributes fa;
      PG_CUDA(cudaFuncGetAttributes(&fa, moe_gemm_kernel));
      g_static_smem = (int)fa.sharedSizeBytes;
      PG_CUDA(cudaFuncSetAttribute(moe_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_max_smem[dev & 63] - g_static_smem));
      g_attr_set[dev & 63] = true;
    }
  }
  MoeGemmParams p;
  memset(&p, 0, sizeof(p));
  p.y = (bf16*)y;
  p.ldy = ldy;
  p.M = M;
  p.K = K;
  p.E = E;
  p.bn = bn;
  p.kblocks = K / BK;
  p.m_tiles = ceil_div(M, BM);
  PG_REQUIRE(quant >= 0 && quant <= 2, "moe gemm: unknown weight storage mode %d", quant);
  PG_REQUIRE(quant == 0 || scales != nullptr, "moe gemm: quantised weights need scales");
  p.quant = quant;
  p.scales = scales;
  p.offsets = (const int*)offsets;
  p.status = (uint32_t*)status;
  p.scatter_src = (const int*)scatter_src;
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
  const int stage_bytes = A_BYTES + bn * 128 + (quant == 1 ? RAW_BYTES : quant == 2 ? RAW_BYTES_FP8 : 0);
  const int tail = (3 * MAX_STAGES + 4) * 8 + 64;
  p.stages = (g_max_smem[dev & 63] - g_static_smem - 1024 - tail) / stage_bytes;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  if (quant) {
    // The four dequant groups take k-blocks 0,1,2,3 (mod 4).  With a stage count that is a
    // multiple of 4 every stage barrier is only ever waited on by one group, in order; any other
    // count lets a group wait on a barrier that is still two phases behind, and a parity wait
    // cannot tell that from "done".
    p.stages -= p.stages % 4;
    PG_REQUIRE(p.stages >= 4, "moe gemm: token tile %d leaves fewer than 4 pipeline stages for quantised weights", bn);
  }
  PG_REQUIRE(p.stages >= 2, "moe gemm: not enough shared memory");
  uint32_t cols = 32;
  while (cols < (uint32_t)(2 * bn)) cols <<= 1;
  p.tmem_cols = cols;

  CUtensorMap tm_w, tm_x;
  cuuint32_t estr[3] = {1, 1, 1};
  if (quant == 2) {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)M * K};
    cuuint32_t box[3] = {BK, BM, 1};
    CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PG_REQUIRE(r == CUDA_SUCCESS, "moe gemm: fp8 weight tensor map failed (%d)", (int)r);
  } else if (quant == 1) {
    cuuint64_t dims[3] = {(cuuint64_t)(K / 8), (cuuint64_t)M, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)(K / 8) * 4, (cuuint64_t)M * (K / 8) * 4};
    cuuint32_t box[3] = {BK / 8, BM, 1};
    CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PG_REQUIRE(r == CUDA_SUCCESS, "moe gemm: packed weight tensor map failed (%d)", (int)r);
  } else {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)M * K * 2};
    cuuint32_t box[3] = {BK, BM, 1};
    CUresult r = enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PG_REQUIRE(r == CUDA_SUCCESS, "moe gemm: weight tensor map failed (%d)", (int)r);
  }
  int rc = pg_make_tmap_bf16_2d(&tm_x, x, x_rows, K, ldx, bn, BK);
  if (rc) return rc;
  const size_t smem = 1024 + (size_t)p.stages * stage_bytes + tail;
  moe_gemm_kernel<<<g_sms[dev & 63], quant ? 448 : 192, smem, stream>>>(tm_w, tm_x, p);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_moe_grouped_gemm(const void* x, long long ldx, long long x_rows, const void* w, const void* scales, int quant, void* y,
                                   long long ldy, const void* offsets, int E, int M, int K, int bn, void* status, cudaStream_t stream) {
  return moe_gemm_impl(x, ldx, x_rows, w, scales, quant, y, ldy, offsets, E, M, K, bn, status, nullptr, nullptr, nullptr, 0, 0, 1, 0, stream);
}

// Expert-parallel W2: output rows are stored straight into their source ranks' combine
// buffers (row stride ldy) and the kernel's tail raises this rank's "returned" epoch.
extern "C" int pg_moe_grouped_gemm_return(const void* x, long long ldx, long long x_rows, const void* w, const void* scales, int quant, long long ldy,
                                          const void* offsets, int E, int M, int K, int bn, void* status, const void* scatter_src,
                                          void* const* peer_out, void* const* peer_flags, int cap, int rank, int world, int site,
                                          cudaStream_t stream) {
  PG_REQUIRE(scatter_src != nullptr && world >= 1 && world <= 8, "moe gemm return: needs the sorted-source table and 1..8 ranks");
  return moe_gemm_impl(x, ldx, x_rows, w, scales, quant, nullptr, ldy, offsets, E, M, K, bn, status, scatter_src, peer_out, peer_flags, cap, rank, world,
                       site, stream);
}
