// bf16 GEMM  Y[T, M] = X[T, K] * W[M, K]^T  on tcgen05 tensor cores.
//
// The weight matrix is the UMMA "A" operand (128 rows of W per tile fill the MMA M
// dimension) and the token rows are the "B" operand (N = token tile, 16..256), so a
// decode step with a handful of tokens still issues full-width 128-row MMAs and simply
// streams W through shared memory once: the kernel is HBM-bound for small T and
// tensor-bound for large T with the same code.
//
//   warp 0      TMA producer: W tile [128 x 64] and X tile [bn x 64] per stage
//   warp 1      allocates TMEM, issues tcgen05.mma (one thread), commits to mbarriers
//   warps 2..5  epilogue: tcgen05.ld the f32 accumulator (one TMEM lane = one W row per
//               thread), convert, store; two accumulator buffers so the epilogue of one
//               tile overlaps the main loop of the next
//
// Persistent grid, static round-robin over work items (tile, k-split).  With k-splits,
// every split writes an f32 partial into a workspace and bumps a per-tile counter; the
// CTA that arrives last sums the partials in split order (deterministic) and writes the
// output, then re-arms the counter, so the workspace needs no clearing between launches.
//
// Takes the place of the reference's cuBLAS/cuBLASLt layer
// (pegainfer-kernels/csrc/shared/linear.cu:294-596).
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int MAX_STAGES = 12;

struct GemmParams {
  bf16* y;
  float* y_f32;
  long long ldy;
  int M, T, K;
  int bn;
  int m_tiles, n_tiles, kblocks, splits;
  int stages;
  uint32_t tmem_cols;
  float* ws;
  uint32_t* counters;
  uint32_t* status;
};

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

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  const int stage_bytes = A_BYTES + p.bn * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tfull = empty + MAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* last_flag = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total = p.m_tiles * p.n_tiles * p.splits;

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
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int tile = item / p.splits, s = item - tile * p.splits;
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
        const int kb0 = (int)(((long long)p.kblocks * s) / p.splits);
        const int kb1 = (int)(((long long)p.kblocks * (s + 1)) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = tiles + stage * stage_bytes;
          mbar_expect_tx(&full[stage], (uint32_t)stage_bytes);
          tma_load_2d(a_dst, &tm_w, &full[stage], kb * BK, m_tile * BM, pol_w);
          tma_load_2d(a_dst + A_BYTES, &tm_x, &full[stage], kb * BK, n_tile * p.bn, pol_x);
          used[stage] = true;
          last_phase[stage] = phase;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Drain: every bulk copy this thread issued must have landed before the CTA exits.
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
        const int tile = item / p.splits, s = item - tile * p.splits;
        const int kb0 = (int)(((long long)p.kblocks * s) / p.splits);
        const int kb1 = (int)(((long long)p.kblocks * (s + 1)) / p.splits);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.bn);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16_ss(d_tmem, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
          }
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
  } else {
    // epilogue: warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int et = threadIdx.x - 64;  // 0..127 among epilogue threads
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      const int tile = item / p.splits, s = item - tile * p.splits;
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      bool ok = mbar_wait(&tfull[acc], acc_phase, abort_flag);
      ok = named_bar_all(1, 128, ok);
      if (!ok) break;
      tc_fence_after();
      const int m = m_tile * BM + r;
      const int n0 = n_tile * p.bn;
      const uint32_t t_row = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(acc * p.bn);
      float* ws_part = p.ws + ((size_t)(tile * p.splits + s) * p.bn) * BM + r;
      for (int c = 0; c < p.bn; c += 16) {
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
        if (p.splits == 1) {
          if (m < p.M) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = n0 + c + j;
              if (n < p.T) {
                if (p.y_f32)
                  p.y_f32[(size_t)n * p.ldy + m] = __uint_as_float(v[j]);
                else
                  p.y[(size_t)n * p.ldy + m] = __float2bfloat16(__uint_as_float(v[j]));
              }
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) ws_part[(size_t)(c + j) * BM] = __uint_as_float(v[j]);
        }
      }
      // accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

      if (p.splits > 1) {
        __threadfence();
        named_bar_all(1, 128, true);
        if (et == 0) {
          const uint32_t old = atomicAdd(&p.counters[tile], 1u);
          *last_flag = (old == (uint32_t)(p.splits - 1)) ? 1u : 0u;
        }
        named_bar_all(1, 128, true);
        if (*last_flag) {
          __threadfence();
          const float* ws_tile = p.ws + ((size_t)tile * p.splits * p.bn) * BM + r;
          const int nmax = min(p.bn, p.T - n0);
          // 16 columns at a time, four splits' loads in flight together: the loop is
          // bound by L2 latency, so independent loads must not be serialised by stores
          for (int c = 0; c < nmax; c += 16) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            for (int q0 = 0; q0 < p.splits; q0 += 4) {
              float tmp[4][16];
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
                const bool live = q0 + qq < p.splits;
                const float* src = ws_tile + ((size_t)(live ? q0 + qq : q0) * p.bn + c) * BM;
#pragma unroll
                for (int j = 0; j < 16; ++j) tmp[qq][j] = live ? __ldcg(src + (size_t)j * BM) : 0.f;
              }
#pragma unroll
              for (int qq = 0; qq < 4; ++qq) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += tmp[qq][j];
              }
            }
            if (m < p.M) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int n = c + j;
                if (n < nmax) {
                  if (p.y_f32)
                    p.y_f32[(size_t)(n0 + n) * p.ldy + m] = acc[j];
                  else
                    p.y[(size_t)(n0 + n) * p.ldy + m] = __float2bfloat16(acc[j]);
                }
              }
            }
          }
          if (et == 0) p.counters[tile] = 0u;
        }
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
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (1u << 8));
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

struct DeviceInfo {
  int sms = 0;
  int max_smem = 0;
  bool attr_set = false;
};
DeviceInfo g_dev[64];
std::mutex g_mu;

}  // namespace

// Row-major [rows, cols] bf16 matrix with row stride ld elements; box = [box_rows x 64].
int pg_make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols) {
  EncodeTiledFn enc = get_encode();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0, "TMA base address must be 16-byte aligned");
  PG_REQUIRE((ld * 2) % 16 == 0, "TMA row stride must be a multiple of 16 bytes (ld=%lld)", ld);
  PG_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_cols * 2 == 128, "unsupported TMA box %dx%d", box_rows, box_cols);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}

static int pick_bn(int T, int M, int sms) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  // large T: time ~ waves x (MMA time ~ bn, plus the fixed 128-row weight tile per stage)
  const int m_tiles = ceil_div(M, BM);
  int best = 256;
  long long best_cost = -1;
  for (int bn = 256; bn >= 128; bn -= 16) {
    const long long tiles = (long long)m_tiles * ceil_div(T, bn);
    const long long waves = (tiles + sms - 1) / sms;
    const long long cost = waves * (bn + 64);
    if (best_cost < 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

// Pick the k-split count that minimises (wave quantisation) x (partial-sum overhead).
static int pick_splits(int tiles, int kblocks, int bn, int sms) {
  if (tiles >= 4 * sms) return 1;
  if (bn > 64 && tiles * 2 > sms) return 1;  // wide tiles: the f32 partial round trip costs more than the idle SMs
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && kblocks / s < 4) break;
    long long items = (long long)tiles * s;
    long long waves = (items + sms - 1) / sms;
    double eff = (double)items / (double)(waves * sms);
    // a split adds 2 * bn * 128 * 4 bytes of L2 traffic per item on top of kblocks/s * 16 KB of weights
    double overhead = s > 1 ? (2.0 * bn * 128 * 4) / ((double)kblocks / s * A_BYTES) : 0.0;
    double cost = (1.0 + 0.5 * overhead) / eff;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

extern "C" int pg_gemm_workspace_bytes(int T, int M, int K, int device, long long* ws_bytes, long long* counter_bytes) {
  int sms = 0;
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  int bn = pick_bn(T, M, sms);
  int tiles = ceil_div(M, BM) * ceil_div(T, bn);
  int splits = pick_splits(tiles, ceil_div(K, BK), bn, sms);
  *ws_bytes = splits > 1 ? (long long)tiles * splits * bn * BM * 4 : 0;
  *counter_bytes = (long long)tiles * 4;
  return PG_OK;
}

// y[T, M] (row stride ldy) = x[T, K] (row stride ldx) * w[M, K]^T (row stride ldw).
// `ws`/`counters` are caller-provided scratch (see pg_gemm_workspace_bytes); the counters
// must be zero before the first use and are left zero by every completed launch.
// `force_splits` > 0 pins the k-split count (batch-invariant serving); 0 = heuristic.
extern "C" int pg_gemm_bf16_tn(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx, long long ldw,
                               long long ldy, void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status,
                               int force_splits, cudaStream_t stream) {
  PG_REQUIRE(T > 0 && M > 0 && K > 0, "gemm: empty problem %dx%dx%d", T, M, K);
  PG_REQUIRE(K % 8 == 0, "gemm: K=%d must be a multiple of 8 (16-byte TMA rows)", K);
  PG_REQUIRE(status != nullptr, "gemm: a device status word is required");
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  DeviceInfo& di = g_dev[dev & 63];
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!di.attr_set) {
      PG_CUDA(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
      PG_CUDA(cudaDeviceGetAttribute(&di.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
      PG_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem));
      di.attr_set = true;
    }
  }
  GemmParams p;
  p.bn = pick_bn(T, M, di.sms);
  p.m_tiles = ceil_div(M, BM);
  p.n_tiles = ceil_div(T, p.bn);
  p.kblocks = ceil_div(K, BK);
  const int tiles = p.m_tiles * p.n_tiles;
  p.splits = force_splits > 0 ? force_splits : pick_splits(tiles, p.kblocks, p.bn, di.sms);
  if (p.splits > p.kblocks) p.splits = p.kblocks;
  if (force_splits <= 0) {
    // never outgrow the caller's scratch: fewer splits only cost load balance
    while (p.splits > 1 && (ws == nullptr || ws_bytes < (long long)tiles * p.splits * p.bn * BM * 4 || counter_bytes < (long long)tiles * 4)) --p.splits;
  }
  if (p.splits > 1) {
    PG_REQUIRE(ws != nullptr && ws_bytes >= (long long)tiles * p.splits * p.bn * BM * 4, "gemm: workspace too small for %d splits", p.splits);
    PG_REQUIRE(counters != nullptr && counter_bytes >= (long long)tiles * 4, "gemm: counter buffer too small");
  }
  const int stage_bytes = A_BYTES + p.bn * 128;
  const int tail = (2 * MAX_STAGES + 4) * 8 + 64;
  p.stages = (di.max_smem - 1024 - tail) / stage_bytes;
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  PG_REQUIRE(p.stages >= 2, "gemm: not enough shared memory for a 2-stage pipeline");
  uint32_t cols = 32;
  while (cols < (uint32_t)(2 * p.bn)) cols <<= 1;
  p.tmem_cols = cols;
  p.y = y_is_f32 ? nullptr : (bf16*)y;
  p.y_f32 = y_is_f32 ? (float*)y : nullptr;
  p.ldy = ldy;
  p.M = M;
  p.T = T;
  p.K = K;
  p.ws = (float*)ws;
  p.counters = (uint32_t*)counters;
  p.status = (uint32_t*)status;
  CUtensorMap tm_w, tm_x;
  int rc = pg_make_tmap_bf16_2d(&tm_w, w, M, K, ldw, BM, BK);
  if (rc) return rc;
  rc = pg_make_tmap_bf16_2d(&tm_x, x, T, K, ldx, p.bn, BK);
  if (rc) return rc;
  const int total = tiles * p.splits;
  const int grid = total < di.sms ? total : di.sms;
  const size_t smem = 1024 + (size_t)p.stages * stage_bytes + tail;
  gemm_bf16_tn_kernel<<<grid, NUM_THREADS, smem, stream>>>(tm_w, tm_x, p);
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// ---------------------------------------------------------------------------------
// Allocation-free variant (see gemm_noalloc.h): same kernel, scratch inside the image.
// ---------------------------------------------------------------------------------
#include "gemm_noalloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer
// that a kernel could be given.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PG_NOALLOC_SCRATCH_BYTES];

static void* g_noalloc_ptr[64];
static bool g_noalloc_ready[64];
static std::mutex g_noalloc_mu;

extern "C" int pg_gemm_bf16_tn_noalloc(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                                       void* status, cudaStream_t stream) {
  PG_REQUIRE(T > 0 && M > 0 && K > 0, "gemm_noalloc: empty problem %dx%dx%d", T, M, K);
  int dev = 0;
  PG_CUDA(cudaGetDevice(&dev));
  PG_REQUIRE(dev >= 0 && dev < 64, "gemm_noalloc: device ordinal %d out of range", dev);
  void* scratch = nullptr;
  int sms = 0;
  {
    // once per device, with that device current: resolve the device address of the array
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ready[dev]) {
      void* ptr = nullptr;
      PG_CUDA(cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch));
      PG_REQUIRE(ptr != nullptr, "gemm_noalloc: scratch symbol resolved to a null address");
      g_noalloc_ptr[dev] = ptr;
      g_noalloc_ready[dev] = true;
    }
    scratch = g_noalloc_ptr[dev];
  }
  PG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int bn = pick_bn(T, M, sms);
  const long long tiles = (long long)ceil_div(M, BM) * ceil_div(T, bn);
  PG_REQUIRE(tiles <= PG_NOALLOC_MAX_TILES,
             "gemm_noalloc: %lld output tiles (M=%d, T=%d) exceed the built-in scratch limit of %d tiles; use pg_gemm_bf16_tn with caller scratch",
             tiles, M, T, (int)PG_NOALLOC_MAX_TILES);
  unsigned char* base = static_cast<unsigned char*>(scratch);
  // the counters must start at zero; the partial sums are fully written before they are read
  PG_CUDA(cudaMemsetAsync(base, 0, (size_t)tiles * 4, stream));
  return pg_gemm_bf16_tn(x, w, y, 0, T, M, K, ldx, ldw, ldy, base + PG_NOALLOC_COUNTER_BYTES,
                         (long long)PG_NOALLOC_SCRATCH_BYTES - PG_NOALLOC_COUNTER_BYTES, base, PG_NOALLOC_COUNTER_BYTES, status, 0, stream);
}
