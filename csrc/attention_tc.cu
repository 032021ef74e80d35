// Prefill attention on tcgen05 for sm_100a: causal GQA attention of ragged query rows over a paged KV cache,
// head dim 128.
//
// One CTA owns 128 query rows of one query head and walks the KV of its sequence in tiles of 128 keys:
//
//   S = Q K^T          tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), accumulator in TMEM
//   P = softmax tile   four warps, one query row per thread: tcgen05.ld of the row, running max / sum in registers,
//                      P written as bf16 into the swizzled A-operand layout
//   O_j = P V          tcgen05.mma with V as an MN-major B operand (the cache stores keys as rows, which is what the
//                      contraction over keys needs transposed), fresh TMEM accumulator per tile
//   O += ...           the row's thread reads O_j back and folds it into its f32 registers with the rescale factor
//
// Roles: warp 0 = TMA producer (Q once, then K and V tiles through the page table, two stages), warp 1 = MMA issuer
// (S of tile j + 1 is issued before P V of tile j, so the tensor core works during the softmax), warps 2-5 = softmax
// and output.  S is double-buffered in TMEM (2 x 128 columns) and O_j takes 128 more.  Every wait is bounded and
// reports through the status word.
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

struct TcSmem {
  uint64_t q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], s_empty[2], p_ready, o_full, o_empty;
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

__global__ void __launch_bounds__(192) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* q_tile = tiles;                       // 32 KB
  uint8_t* p_tile = tiles + TILE_BYTES;          // 32 KB
  uint8_t* k_tile = tiles + 2 * TILE_BYTES;      // 2 x 32 KB
  uint8_t* v_tile = tiles + 4 * TILE_BYTES;      // 2 x 32 KB
  TcSmem* sh = reinterpret_cast<TcSmem*>(tiles + 6 * TILE_BYTES);
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->kv_empty[s], 1);
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->s_empty[s], 4);
    }
    mbar_init(&sh->p_ready, 4);
    mbar_init(&sh->o_full, 1);
    mbar_init(&sh->o_empty, 4);
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
  const uint32_t tmem = sh->tmem_slot;
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
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&sh->kv_empty[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag)) break;
        mbar_expect_tx(&sh->k_full[s], TILE_BYTES);
        mbar_expect_tx(&sh->v_full[s], TILE_BYTES);
        const int pages_live = min(ppt, (kv_len - j * BKV + p.page_size - 1) / p.page_size);
        for (int kvsel = 0; kvsel < 2; ++kvsel) {
          uint8_t* dst = (kvsel ? v_tile : k_tile) + s * TILE_BYTES;
          uint64_t* bar = kvsel ? &sh->v_full[s] : &sh->k_full[s];
          for (int pg = 0; pg < ppt; ++pg) {
            // pages past the sequence's end read page 0 (the padding page): their keys are masked
            long long page = pg < pages_live ? table_row[j * ppt + pg] : 0;
            if (page < 0 || page >= p.num_pages) {
              atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (41u << 8));
              page = 0;
            }
            const int z = (int)((page * 2 + kvsel) * p.page_size);
            tma_load_3d(dst + pg * p.page_size * 128, &tm_kv, bar, 0, h, z, pol);
            tma_load_3d(dst + HALF_BYTES + pg * p.page_size * 128, &tm_kv, bar, 64, h, z, pol);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_o = idesc_bf16(128, 128, 1);
      const uint32_t qa = smem_u32(q_tile), pa = smem_u32(p_tile);
      const uint32_t lbo = p.mn_lbo_first ? (uint32_t)HALF_BYTES : 1024u, sbo = p.mn_lbo_first ? 1024u : (uint32_t)HALF_BYTES;
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait(&sh->k_full[s], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
        if (j >= 2 && !mbar_wait(&sh->s_empty[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(k_tile + s * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + (uint32_t)(s * 128), umma_desc_k_sw128(qa + kb * HALF_BYTES + k * 32), umma_desc_k_sw128(ka + kb * HALF_BYTES + k * 32), idesc_s,
                         (kb | k) ? 1u : 0u);
        umma_commit(&sh->s_full[s]);
        return true;
      };
      ok = ok && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        ok = mbar_wait(&sh->p_ready, (uint32_t)(j & 1), abort_flag) && mbar_wait(&sh->v_full[s], (uint32_t)((j >> 1) & 1), abort_flag);
        if (ok && j >= 1) ok = mbar_wait(&sh->o_empty, (uint32_t)((j - 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(v_tile + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(tmem + 256u, umma_desc_k_sw128(pa + (ks >> 2) * HALF_BYTES + (ks & 3) * 32), umma_desc_mn_sw128(va + ks * 2048, lbo, sbo), idesc_o, ks ? 1u : 0u);
        umma_commit(&sh->o_full);
        umma_commit(&sh->kv_empty[s]);
      }
    }
  } else {
    // softmax / output warps: TMEM lanes 32 * (warp % 4) .., one query row per thread
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int my_pos = pos_base + r;  // rows past rows_here compute garbage that is never stored
    const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    bool ok = true;
    uint8_t* p_row = p_tile + r * 128;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&sh->s_full[s], (uint32_t)((j >> 1) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_row = lane_base + (uint32_t)(s * 128);
      const int key0 = j * BKV;
      const bool need_mask = key0 + BKV - 1 > min(pos_base, kv_len - 1);
      const int limit = min(my_pos, kv_len - 1) - key0;  // keys 0 .. limit of this tile are visible
      // pass 1: row maximum
      float mx = m;
#pragma unroll
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld32(s_row + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float x = __uint_as_float(v[i]) * p.scale_log2;
          if (!need_mask || c + i <= limit) mx = fmaxf(mx, x);
        }
      }
      const float alpha = (mx == -INFINITY) ? 1.f : exp2f(m - mx);  // m = -inf gives 0
      // the previous tile's P V product: fold it in before P is overwritten
      if (j >= 1) {
        ok = mbar_wait(&sh->o_full, (uint32_t)((j - 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_base + 256u + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] = fmaf(o[c + i], alpha_prev, __uint_as_float(v[i]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->o_empty);
      }
      // pass 2: P = exp2(S - max), row sum, bf16 into the swizzled A layout
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld32(s_row + c, v);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = 0.f, e1 = 0.f;
          if (!need_mask || c + i <= limit) e0 = exp2f(__uint_as_float(v[i]) * p.scale_log2 - mx);
          if (!need_mask || c + i + 1 <= limit) e1 = exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - mx);
          const bf162 pr = __floats2bfloat162_rn(e0, e1);
          // the sum uses the rounded values the tensor core will see
          sum += __bfloat162float(pr.x) + __bfloat162float(pr.y);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pr);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c >> 3) + q4;  // 16-byte chunk 0..15 of the row (8 keys each)
          *reinterpret_cast<uint4*>(p_row + (chunk >> 3) * HALF_BYTES + (((chunk & 7) ^ (r & 7)) << 4)) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      }
      l = l * alpha + sum;
      m = mx;
      alpha_prev = 1.f;  // O so far is rescaled by the NEXT tile's alpha when that tile's product is folded in
      // o currently holds sum_{i<j} with the scale of tile j-1's max: bring it to the new max now
      if (alpha != 1.f) {
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] *= alpha;
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sh->s_empty[s]);
        mbar_arrive(&sh->p_ready);
      }
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&sh->o_full, (uint32_t)((n_tiles - 1) & 1), abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_base + 256u + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] += __uint_as_float(v[i]);
        }
      }
    }
    if (r < rows_here) {
      const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
      bf16* dst = p.out + ((long long)(q0 + row_base + r) * p.hq + hq) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = o[c + i] * inv;
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
  const size_t smem = 1024 + 6 * (size_t)TILE_BYTES + sizeof(TcSmem) + 64;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(prefill_attn_tc_kernel, dim3((unsigned)q_tiles, (unsigned)hq), dim3(192), smem, stream, tm_q, tm_kv, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
