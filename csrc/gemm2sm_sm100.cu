// bf16 GEMM  Y[T, M] = X[T, K] * W[M, K]^T  for large T: two SMs work on one tile.
//
// A pair of CTAs (a thread-block cluster of 2) computes a 256 (weight rows) x 256 (tokens)
// tile with tcgen05.mma.cta_group::2.  Each CTA stages only its own half of both operands,
// 128 weight rows and 128 token rows per 64-deep k-block, so a stage is 32 KB per CTA for
// 256 x 256 x 64 multiply-adds of the pair.  The one-CTA kernel in gemm_sm100.cu moves
// 48 KB per CTA for 128 x 256 x 64: per multiply-add this kernel writes and reads a third
// as many shared-memory bytes, which is what limits the one-CTA kernel at large T (TMA
// writes plus operand reads exceed what one SM's shared memory delivers per clock at full
// tensor rate).  The accumulator of each CTA is its 128 rows x 256 columns of the tile in
// its own TMEM, two buffers, so the epilogue of a tile overlaps the main loop of the next.
//
//   CTA rank 0 (leader)                          CTA rank 1
//   warp 0  TMA producer (own halves)            warp 0  TMA producer (own halves)
//   warp 1  TMEM alloc, issues every MMA          warp 1  TMEM alloc / dealloc only
//   warps 2..5 epilogue of rows 0..127            warps 2..5 epilogue of rows 128..255
//
// Barriers: `full[s]` lives in the leader and counts the bytes of BOTH CTAs' loads (each
// CTA's TMA names the leader's barrier); `empty[s]` and `tfull[a]` exist in both CTAs and
// are signalled by tcgen05.commit with a two-CTA multicast mask; `tempty[a]` lives in the
// leader and counts the eight epilogue warps of the pair.  Every wait is bounded.
//
// Takes the place of the reference's cuBLAS/cuBLASLt layer for prefill-sized problems
// (pegainfer-kernels/csrc/shared/linear.cu:294-596).
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128;  // weight rows per CTA (256 per pair)
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 12;
constexpr int NUM_THREADS = 192;
constexpr int RASTER_GROUP = 8;  // weight-row pairs per raster group

struct Gemm2Params {
  bf16* y;
  long long ldy;
  int M, T, K;
  int m_pairs, n_tiles, kblocks;
  int bn;      // token columns of a pair's tile (multiple of 32, <= 256); each CTA stages bn / 2 token rows
  int stages;  // shared-memory ring depth
  uint32_t tmem_cols;
  uint32_t* status;
  int epi;  // 0: y = x W^T; 1: the weight rows alternate (gate_i, up_i) and y [T, M / 2] = bf16(silu(gate)) * up
};

// Work item -> (weight-row pair, token tile).  Items walk RASTER_GROUP weight-row pairs across
// all token tiles before moving on, so the CTA pairs that run at the same time cover a
// near-square patch of the output and share both operands through L2 (walking all weight
// rows of one token tile first would stream the whole weight matrix once per token tile).
__device__ __forceinline__ void tile_of(const Gemm2Params& p, int item, int& m_pair, int& n_tile) {
  const int per_group = RASTER_GROUP * p.n_tiles;
  const int group = item / per_group;
  const int first = group * RASTER_GROUP;
  const int gsz = min(RASTER_GROUP, p.m_pairs - first);
  const int within = item - group * per_group;
  m_pair = first + within % gsz;
  n_tile = within / gsz;
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem of both CTAs]; one thread of the leader.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in every CTA of `mask` once all MMAs
// issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}
// Tiled load into this CTA's shared memory; the bytes are counted on `bar_cluster_addr`,
// a barrier that may live in the other CTA of the pair.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2sm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  const int bnh = p.bn >> 1;
  const int stage_bytes = A_BYTES + bnh * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, p.tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrive or multicast commit
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();
  pdl_wait();

  const int total = p.m_pairs * p.n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      // both operands are re-read (weights by every token tile, tokens by every weight-row pair)
      const uint64_t pol_w = l2_policy_evict_normal();
      const uint64_t pol_x = l2_policy_evict_normal();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t last_phase[MAX_STAGES];
      bool used[MAX_STAGES];
#pragma unroll
      for (int s = 0; s < MAX_STAGES; ++s) {
        used[s] = false;
        last_phase[s] = 0;
      }
      bool ok = true;
      for (int item = pair; item < total && ok; item += pairs) {
        int m_pair, n_tile;
        tile_of(p, item, m_pair, n_tile);
        const int w_row = m_pair * (2 * BM) + (int)rank * BM;
        const int x_row = n_tile * p.bn + (int)rank * bnh;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_cluster(&empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = tiles + stage * stage_bytes;
          const uint32_t bar = dsmem_addr(smem_u32(&full[stage]), 0u);
          if (rank == 0) mbar_expect_tx(&full[stage], 2u * (uint32_t)stage_bytes);
          tma_load_2d_pair(a_dst, &tm_w, bar, kb * BK, w_row, pol_w);
          tma_load_2d_pair(a_dst + A_BYTES, &tm_x, bar, kb * BK, x_row, pol_x);
          used[stage] = true;
          last_phase[stage] = phase;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Drain: the MMAs that read this CTA's stages have completed (so the loads have landed and
      // the leader's multicast arrivals on this CTA's barriers are in) before the CTA may exit.
      for (int s = 0; s < p.stages; ++s) {
        if (!used[s]) continue;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait_cluster(&empty[s], last_phase[s])) {
          if (*abort_flag || globaltimer_ns() - t0 > PG_WAIT_LIMIT_NS) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(2 * BM, (uint32_t)p.bn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = pair; item < total && ok; item += pairs) {
        if (!mbar_wait_cluster(&tempty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_cluster(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16_ss_pair(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], (uint16_t)3);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[acc], (uint16_t)3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31 of its own CTA
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int item = pair; item < total; item += pairs) {
      int m_pair, n_tile;
      tile_of(p, item, m_pair, n_tile);
      if (!mbar_wait_cluster(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const int m = m_pair * (2 * BM) + (int)rank * BM + r;
      const int n0 = n_tile * p.bn;
      const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * p.bn);
      bf16* yc = p.y + m;
      for (int c = 0; c < p.bn; c += 32) {
        uint32_t v[2][16];
        tmem_ld16(t_row + c, v[0]);
        tmem_ld16(t_row + c + 16, v[1]);
        tmem_ld_wait();
        if (p.epi == 1) {
          // SwiGLU: lanes 2 i and 2 i + 1 hold gate and up of output column m / 2 (both rounded to bf16 first, as the
          // separate kernel sees them); the shuffles run on all lanes, the even ones store
          bf16* ys = p.y + (m >> 1);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float mine = __bfloat162float(__float2bfloat16(__uint_as_float(v[h][j])));
              const float other = __shfl_xor_sync(0xFFFFFFFFu, mine, 1);
              const int n = n0 + c + h * 16 + j;
              if (!(lane & 1) && m < p.M && n < p.T) {
                const float a = __bfloat162float(__float2bfloat16(mine / (1.f + __expf(-mine))));
                ys[(long long)n * p.ldy] = __float2bfloat16(a * other);
              }
            }
          }
        } else if (m < p.M) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = n0 + c + h * 16 + j;
              if (n < p.T) yc[(long long)n * p.ldy] = __float2bfloat16(__uint_as_float(v[h][j]));
            }
          }
        }
      }
      // this accumulator buffer may be overwritten: tell the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(dsmem_addr(smem_u32(&tempty[acc]), 0u));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA tears down shared memory or TMEM the other may still reach
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (11u << 8));
}

std::mutex g_mu2;
struct Dev2 {
  bool set = false;
  bool usable = false;
  int sms = 0;
  int max_smem = 0;
  int max_pairs = 0;
};
Dev2 g_dev2[64];
int g_enabled = -1;

}  // namespace

// 1 if the two-SM kernel would take this problem on the current device.
extern "C" int pg_gemm2sm_eligible(int T, int M, int K) {
  if (g_enabled < 0) {
    const char* e = getenv("PEGAINFER_GEMM_2SM");
    g_enabled = (e && e[0] == '0') ? 0 : 1;
  }
  if (!g_enabled) return 0;
  // Tensor-bound problems with at least about one full round of CTA pairs: below that the
  // one-CTA kernel's narrower token tiles and k-splits fill the machine better.  Very deep
  // problems (K > 8192) stay on the one-CTA kernel as well: there the operand slabs that the
  // concurrently running 256 x 256 tiles share (17 slabs of 256 x K) approach the L2 capacity
  // and this kernel measured slower (493 vs 372 us at T = M = 4096, K = 12288).
  static int max_k = 0;
  if (max_k == 0) {
    const char* e = getenv("PEGAINFER_GEMM_2SM_MAXK");
    max_k = e ? atoi(e) : 8192;
    if (max_k <= 0) max_k = 8192;
  }
  if (T < 256 || M < 1024 || K < 256 || K > max_k || K % 8 != 0) return 0;
  return (long long)ceil_div(M, 2 * BM) * ceil_div(T, 256) >= 64 ? 1 : 0;
}

static int gemm2sm_impl(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status, int epi, cudaStream_t stream);

extern "C" int pg_gemm2sm_bf16_tn(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status,
                                  cudaStream_t stream) {
  return gemm2sm_impl(x, w, y, T, M, K, ldx, ldw, ldy, status, 0, stream);
}

// The same product with SwiGLU in the epilogue: w [M, K] with rows alternating (gate_i, up_i), y [T, M / 2].
extern "C" int pg_gemm2sm_bf16_tn_swiglu(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status,
                                         cudaStream_t stream) {
  PG_REQUIRE(M % 2 == 0, "gemm2sm swiglu: M %d must be even (interleaved gate / up rows)", M);
  return gemm2sm_impl(x, w, y, T, M, K, ldx, ldw, ldy, status, 1, stream);
}

static int gemm2sm_impl(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status, int epi, cudaStream_t stream) {
  PG_REQUIRE(T > 0 && M > 0 && K > 0 && K % 8 == 0, "gemm2sm: bad problem %dx%dx%d", T, M, K);
  PG_REQUIRE(status != nullptr, "gemm2sm: a device status word is required");
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  Dev2& di = g_dev2[dev & 63];
  const int tail = (2 * MAX_STAGES + 4) * 8 + 64;
  {
    std::lock_guard<std::mutex> lk(g_mu2);
    if (!di.set) {
      PG_CUDA(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
      PG_CUDA(cudaDeviceGetAttribute(&di.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      PG_CUDA(cudaFuncSetAttribute(gemm2sm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3((unsigned)(2 * di.sms));
      cfg.blockDim = dim3(NUM_THREADS);
      cfg.dynamicSmemBytes = (size_t)di.max_smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm2sm_bf16_tn_kernel, &cfg) == cudaSuccess) di.max_pairs = n;
      else (void)cudaGetLastError();
      di.usable = di.max_pairs > 0;
      di.set = true;
    }
  }
  PG_REQUIRE(di.usable, "gemm2sm: no co-resident CTA pair on this device");
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.y = (bf16*)y;
  p.ldy = ldy;
  p.M = M;
  p.T = T;
  p.K = K;
  p.m_pairs = ceil_div(M, 2 * BM);
  // token-tile width: fewest rounds of CTA pairs; a round costs about (width + 256): the MMA
  // time follows the width, the 128 weight rows per CTA and the per-k-block hand-offs do not
  {
    long long best_cost = -1;
    for (int bn = 256; bn >= 128; bn -= 32) {
      const long long tiles = (long long)p.m_pairs * ceil_div(T, bn);
      const long long rounds = (tiles + di.max_pairs - 1) / di.max_pairs;
      const long long cost = rounds * (bn + 256);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        p.bn = bn;
      }
    }
  }
  p.n_tiles = ceil_div(T, p.bn);
  p.kblocks = ceil_div(K, BK);
  const int stage_bytes = A_BYTES + (p.bn / 2) * 128;
  p.stages = (di.max_smem - 1024 - tail) / stage_bytes;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  PG_REQUIRE(p.stages >= 2, "gemm2sm: not enough shared memory");
  p.tmem_cols = 2 * p.bn > 256 ? 512u : 256u;
  p.status = (uint32_t*)status;
  p.epi = epi;
  const size_t smem = 1024 + (size_t)p.stages * stage_bytes + tail;
  CUtensorMap tm_w, tm_x;
  int rc = pg_make_tmap_bf16_2d(&tm_w, w, M, K, ldw, BM, BK);
  if (rc) return rc;
  rc = pg_make_tmap_bf16_2d(&tm_x, x, T, K, ldx, p.bn / 2, BK);
  if (rc) return rc;
  const int total = p.m_pairs * p.n_tiles;
  const int npairs = total < di.max_pairs ? total : di.max_pairs;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(2 * npairs));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int na = 0;
  at[na].id = cudaLaunchAttributeClusterDimension;
  at[na].val.clusterDim.x = 2;
  at[na].val.clusterDim.y = 1;
  at[na].val.clusterDim.z = 1;
  ++na;
  if (pdl_enabled()) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = (unsigned)na;
  PG_CUDA(cudaLaunchKernelEx(&cfg, gemm2sm_bf16_tn_kernel, tm_w, tm_x, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
