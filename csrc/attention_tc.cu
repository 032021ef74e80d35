// Prefill attention on tcgen05 for sm_100a: causal GQA attention of ragged query rows over a paged KV cache,
// head dim 128.
//
// One CTA owns 128 query rows of one query head and walks the KV of its sequence in tiles of 128 keys:
//
//   S = Q K^T          tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), accumulator in TMEM
//   P = softmax tile   eight warps, two threads per query row (64 key columns each): tcgen05.ld of the half row, the two
//                      halves' maxima meet through shared memory, running max / sum in registers, P written as bf16
//                      into the swizzled A-operand layout
//   O_j = P V          tcgen05.mma with V as an MN-major B operand (the cache stores keys as rows, which is what the
//                      contraction over keys needs transposed), fresh TMEM accumulator per tile (two, ping-pong)
//   O += ...           each thread reads its 64 output columns of O_j back and folds them into f32 registers with the
//                      rescale factor of the next tile
//
// Roles: warp 0 = TMA producer (Q once, then K and V tiles through the page table, a ring of four tiles), warp 1 = MMA
// issuer (S of tile j + 1 is issued before P V of tile j, so the tensor core works during the softmax), warps 2-9 =
// softmax and output.  TMEM: S twice 128 columns, O_j twice 128 columns.  Every wait is bounded and reports through
// the status word.
//
// Reference parity: the reference's prefill attention is FlashInfer's BatchPrefillWithPagedKVCache
// (pegainfer-kernels/csrc/shared/flashinfer_prefill.cu), an mma.sync kernel on every architecture.
#include "common.cuh"

#include <cuda.h>

#include <mutex>

namespace {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KB: [2 blocks of 64 columns][128 rows][128 B]
constexpr int HALF_BYTES = TILE_BYTES / 2;

struct TcAttnParams {
  bf16* out;              // [T, hq * D]
  const int* q_indptr;    // [num_seqs + 1]
  const int* kv_lens;     // [num_seqs]
  const int* table;       // [num_seqs, table_stride]
  int table_stride, num_seqs, hq, hkv, page_size;
  long long num_pages;
  float scale_log2;       // softmax scale * log2(e)
  int mn_lbo_first;       // descriptor variant of the MN-major operand (1: LBO = stride between 64-column blocks)
  uint32_t* status;
};

constexpr int RING = 4;           // K / V tiles in flight: K_j, V_j, K_{j+1}, V_{j+1} share one ring
constexpr int SM_WARPS = 8;       // softmax warps: two per TMEM lane quadrant, each thread owns half of a row
constexpr int THREADS = 64 + SM_WARPS * 32;

struct TcSmem {
  uint64_t q_full, kv_full[RING], kv_empty[RING], s_full[2], s_empty[2], p_ready[2], o_full[2], o_empty[2];
  float xmax[2][2][BQ];  // [tile parity][column half][row]: the halves' row maxima
  float xsum[2][BQ];
  uint32_t tmem_slot;
  int abort_flag;
};

// MN-major operand (rows = contraction index, 128-byte rows of 64 consecutive N elements, 128-byte swizzle):
// `lbo` = byte stride between blocks of 64 N elements, `sbo` = byte stride between groups of 8 contraction rows.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> f32, A K-major, B K-major or MN-major
__host__ __device__ constexpr uint32_t idesc_bf16(uint32_t m, uint32_t n, uint32_t b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  tmem_ld16(taddr, r);
  tmem_ld16(taddr + 16, r + 16);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, %0;" ::"n"(SM_WARPS * 32) : "memory"); }

__global__ void __launch_bounds__(THREADS) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* q_tile = tiles;                       // 32 KB
  uint8_t* p_tile = tiles + TILE_BYTES;          // 32 KB
  uint8_t* ring = tiles + 2 * TILE_BYTES;        // RING x 32 KB
  TcSmem* sh = reinterpret_cast<TcSmem*>(tiles + (2 + RING) * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = blockIdx.y;
  const int h = hq / (p.hq / p.hkv);

  // (sequence, query tile) of this CTA: late tiles (most keys) first
  int b = 0, tile_in_seq = 0;
  {
    int rem = (int)gridDim.x - 1 - (int)blockIdx.x;
    for (; b < p.num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + BQ - 1) / BQ;
      if (rem < nt) {
        tile_in_seq = rem;
        break;
      }
      rem -= nt;
    }
    if (b >= p.num_seqs) return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->s_empty[s], SM_WARPS);
      mbar_init(&sh->p_ready[s], SM_WARPS);
      mbar_init(&sh->o_full[s], 1);
      mbar_init(&sh->o_empty[s], SM_WARPS);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_kv);
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;  // columns: S0 0..127, S1 128..255, O0 256..383, O1 384..511
  volatile int* abort_flag = &sh->abort_flag;
  PG_PDL_ENTRY();

  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int row_base = tile_in_seq * BQ;
  const int rows_here = min(BQ, q_len - row_base);
  const int pos_base = kv_len - q_len + row_base;                 // position of the tile's first row
  const int last_pos = pos_base + rows_here - 1;                  // last key any row of the tile may see
  const int n_tiles = kv_len > 0 ? min(last_pos, kv_len - 1) / BKV + 1 : 0;
  const int* table_row = p.table + (long long)b * p.table_stride;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      const uint64_t pol = l2_policy_evict_normal();
      mbar_expect_tx(&sh->q_full, TILE_BYTES);
      tma_load_3d(q_tile, &tm_q, &sh->q_full, 0, hq, q0 + row_base, pol);
      tma_load_3d(q_tile + HALF_BYTES, &tm_q, &sh->q_full, 64, hq, q0 + row_base, pol);
      const int ppt = BKV / p.page_size;  // pages per key tile
      // load n = 2 j (K of tile j) or 2 j + 1 (V of tile j) goes to ring slot n % RING.  The tile's page ids are
      // read in one unrolled burst (independent loads in flight together); read one by one between the TMA issues,
      // each would cost a full memory latency and the page walk alone would take longer than the tile's MMAs.
      int pages[16];
      for (int n = 0; n < 2 * n_tiles; ++n) {
        const int j = n >> 1, kvsel = n & 1, slot = n % RING, use = n / RING;
        if (kvsel == 0) {
          const int pages_live = min(ppt, (kv_len - j * BKV + p.page_size - 1) / p.page_size);
#pragma unroll
          for (int pg = 0; pg < 16; ++pg) pages[pg] = (pg < pages_live) ? __ldg(table_row + j * ppt + pg) : 0;  // past the end: the padding page, keys masked
#pragma unroll
          for (int pg = 0; pg < 16; ++pg) {
            if (pages[pg] < 0 || pages[pg] >= p.num_pages) {
              atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (41u << 8));
              pages[pg] = 0;
            }
          }
        }
        if (use >= 1 && !mbar_wait(&sh->kv_empty[slot], (uint32_t)((use - 1) & 1), abort_flag)) break;
        mbar_expect_tx(&sh->kv_full[slot], TILE_BYTES);
        uint8_t* dst = ring + slot * TILE_BYTES;
#pragma unroll
        for (int pg = 0; pg < 16; ++pg) {
          if (pg < ppt) {
            const int z = (pages[pg] * 2 + kvsel) * p.page_size;
            tma_load_3d(dst + pg * p.page_size * 128, &tm_kv, &sh->kv_full[slot], 0, h, z, pol);
            tma_load_3d(dst + HALF_BYTES + pg * p.page_size * 128, &tm_kv, &sh->kv_full[slot], 64, h, z, pol);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_o = idesc_bf16(128, 128, 1);
      const uint32_t qa = smem_u32(q_tile);
      const uint32_t lbo = p.mn_lbo_first ? (uint32_t)HALF_BYTES : 1024u, sbo = p.mn_lbo_first ? 1024u : (uint32_t)HALF_BYTES;
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int s = j & 1, n = 2 * j, slot = n % RING, use = n / RING;
        if (!mbar_wait(&sh->kv_full[slot], (uint32_t)(use & 1), abort_flag)) return false;
        if (j >= 2 && !mbar_wait(&sh->s_empty[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(ring + slot * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + (uint32_t)(s * 128), umma_desc_k_sw128(qa + kb * HALF_BYTES + k * 32), umma_desc_k_sw128(ka + kb * HALF_BYTES + k * 32), idesc_s,
                         (kb | k) ? 1u : 0u);
        umma_commit(&sh->s_full[s]);
        umma_commit(&sh->kv_empty[slot]);  // the K tile is free once S is done
        return true;
      };
      ok = ok && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1, n = 2 * j + 1, slot = n % RING, use = n / RING;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        ok = mbar_wait(&sh->p_ready[s], (uint32_t)((j >> 1) & 1), abort_flag) && mbar_wait(&sh->kv_full[slot], (uint32_t)(use & 1), abort_flag);
        if (ok && j >= 2) ok = mbar_wait(&sh->o_empty[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(ring + slot * TILE_BYTES), pa = smem_u32(p_tile);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(tmem + 256u + (uint32_t)(s * 128), umma_desc_k_sw128(pa + (ks >> 2) * HALF_BYTES + (ks & 3) * 32), umma_desc_mn_sw128(va + ks * 2048, lbo, sbo), idesc_o,
                       ks ? 1u : 0u);
        umma_commit(&sh->o_full[s]);
        umma_commit(&sh->kv_empty[slot]);
      }
    }
  } else {
    // softmax / output warps.  TMEM lanes 32 * (warp % 4) ..: warps w and w + 4 share a quadrant; the first takes key
    // (and output) columns 0..63 of its rows, the second 64..127.
    const int wq = warp & 3, half = (warp - 2) >> 2;
    const int r = wq * 32 + lane;
    const int my_pos = pos_base + r;  // rows past rows_here compute garbage that is never stored
    const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(half * 64);
    float2 o[32];  // packed pairs: the fold and the rescale are f32x2 instructions
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = make_float2(0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&sh->s_full[s], (uint32_t)((j >> 1) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * BKV + half * 64;
      const bool need_mask = j * BKV + BKV - 1 > min(pos_base, kv_len - 1);
      const int limit = min(my_pos, kv_len - 1) - key0;  // columns 0 .. limit of this thread's half are visible
      uint32_t v[64];
      tmem_ld32(lane_base + (uint32_t)(s * 128), v);
      tmem_ld32(lane_base + (uint32_t)(s * 128) + 32, v + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->s_empty[s]);  // S is in registers
      float mx_raw = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i <= limit) mx_raw = fmaxf(mx_raw, __uint_as_float(v[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx_raw = fmaxf(mx_raw, __uint_as_float(v[i]));
      }
      sh->xmax[s][half][r] = mx_raw;
      softmax_bar();
      const float mx = fmaxf(m, fmaxf(sh->xmax[s][0][r], sh->xmax[s][1][r]) * p.scale_log2);
      const float alpha = (mx == -INFINITY) ? 1.f : ex2_approx(m - mx);
      const float neg = (mx == -INFINITY) ? 0.f : -mx;
      // fold in the previous tile's P V product and move to the new maximum; its completion also frees the P tile
      if (j >= 1) {
        const int sp = (j - 1) & 1;
        ok = mbar_wait(&sh->o_full[sp], (uint32_t)(((j - 1) >> 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t w[32];
          tmem_ld32(lane_base + 256u + (uint32_t)(sp * 128) + c, w);
          tmem_ld_wait();
          if (alpha == 1.f) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) o[(c + i) >> 1] = __fadd2_rn(o[(c + i) >> 1], make_float2(__uint_as_float(w[i]), __uint_as_float(w[i + 1])));
          } else {
            const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              o[(c + i) >> 1] = __fmul2_rn(__fadd2_rn(o[(c + i) >> 1], make_float2(__uint_as_float(w[i]), __uint_as_float(w[i + 1]))), a2);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->o_empty[sp]);
      }
      // P = exp2(S * scale - max) as bf16 into this half's 64-key block of the swizzled A tile
      uint8_t* p_row = p_tile + half * HALF_BYTES + r * 128;
      float2 sum2 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), ng2 = make_float2(neg, neg);
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const int col = c8 * 8 + i;
          const float2 t2 = __ffma2_rn(make_float2(__uint_as_float(v[col]), __uint_as_float(v[col + 1])), sc2, ng2);
          float2 e = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
          if (need_mask) {
            if (col > limit) e.x = 0.f;
            if (col + 1 > limit) e.y = 0.f;
          }
          sum2 = __fadd2_rn(sum2, e);
          const bf162 pr = __floats2bfloat162_rn(e.x, e.y);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        *reinterpret_cast<uint4*>(p_row + ((c8 ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      l = l * alpha + sum2.x + sum2.y;
      m = mx;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_ready[s]);
    }
    if (ok && n_tiles > 0) {
      const int sp = (n_tiles - 1) & 1;
      ok = mbar_wait(&sh->o_full[sp], (uint32_t)(((n_tiles - 1) >> 1) & 1), abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t w[32];
          tmem_ld32(lane_base + 256u + (uint32_t)(sp * 128) + c, w);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) o[(c + i) >> 1] = __fadd2_rn(o[(c + i) >> 1], make_float2(__uint_as_float(w[i]), __uint_as_float(w[i + 1])));
        }
      }
    }
    sh->xsum[half][r] = l;
    softmax_bar();
    if (r < rows_here) {
      const float lt = sh->xsum[0][r] + sh->xsum[1][r];
      const float inv = (ok && lt > 0.f) ? 1.f / lt : 0.f;
      bf16* dst = p.out + ((long long)(q0 + row_base + r) * p.hq + hq) * D + half * 64;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          f[i] = o[(c + i) >> 1].x * inv;
          f[i + 1] = o[(c + i) >> 1].y * inv;
        }
        *reinterpret_cast<bf16x8*>(dst + c) = pack8(f);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0 && sh->abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (41u << 8));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_attn() {
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

// [rows, heads, 128] bf16, contiguous; box = 64 columns x 1 head x box_rows rows, 128-byte swizzle
int make_tmap_rows_heads(CUtensorMap* out, const void* ptr, long long rows, int heads, int box_rows) {
  EncodeTiledFn enc = get_encode_attn();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0, "TMA base address must be 16-byte aligned");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)heads * D * 2};
  cuuint32_t box[3] = {64u, 1u, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}

int g_mn_variant = -1;

}  // namespace

// Test hook: which of the two stride fields of the MN-major descriptor carries the 64-column block stride.
extern "C" void pg_prefill_attention_tc_variant(int v) { g_mn_variant = v; }

// q [T, hq, 128] bf16 (contiguous), kv_layer [pages, 2, page_size, hkv, 128], out [T, hq * 128].  `q_tiles` = sum over the
// sequences of ceil(query rows / 128).
extern "C" int pg_prefill_attention_tc(const void* q, const void* kv_layer, void* out, const void* q_indptr, const void* kv_lens, const void* table, int table_stride,
                                       int num_seqs, int tokens, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int q_tiles, void* status,
                                       cudaStream_t stream) {
  PG_REQUIRE(dim == D, "tcgen05 prefill attention is built for head dim 128 (got %d)", dim);
  PG_REQUIRE(page_size >= 8 && page_size <= 128 && BKV % page_size == 0, "page size %d does not tile 128 keys", page_size);
  PG_REQUIRE(num_pages * 2 * page_size < (1ll << 31), "KV cache of %lld pages is too large for 32-bit TMA row coordinates", num_pages);
  PG_REQUIRE(hq % hkv == 0, "query heads %d are not a multiple of the KV heads %d", hq, hkv);
  if (q_tiles == 0 || tokens == 0) return PG_OK;
  CUtensorMap tm_q, tm_kv;
  int rc = make_tmap_rows_heads(&tm_q, q, tokens, hq, BQ);
  if (rc != PG_OK) return rc;
  rc = make_tmap_rows_heads(&tm_kv, kv_layer, num_pages * 2 * page_size, hkv, page_size);
  if (rc != PG_OK) return rc;
  TcAttnParams p;
  p.out = (bf16*)out;
  p.q_indptr = (const int*)q_indptr;
  p.kv_lens = (const int*)kv_lens;
  p.table = (const int*)table;
  p.table_stride = table_stride;
  p.num_seqs = num_seqs;
  p.hq = hq;
  p.hkv = hkv;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mn_lbo_first = g_mn_variant < 0 ? 1 : g_mn_variant;
  p.status = (uint32_t*)status;
  const size_t smem = 1024 + (2 + RING) * (size_t)TILE_BYTES + sizeof(TcSmem) + 64;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(prefill_attn_tc_kernel, dim3((unsigned)q_tiles, (unsigned)hq), dim3(THREADS), smem, stream, tm_q, tm_kv, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
