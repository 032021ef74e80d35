// Sparse-attention indexer (GLM-5 / DeepSeek-V3.2 style "DSA") for sm_100a.
//
//   pg_dsa_k_append   LayerNorm + rotary on the index key of every row, appended to the paged index cache
//   pg_dsa_q_rope     rotary on the index queries, in place
//   pg_dsa_scores     score[t, j] = sum_h w[t, h] * relu(q[t, h] . k[j]) on the tensor cores: the 128 keys of
//                     a tile are the M rows of one tcgen05.mma chain (K = head dim), the query heads its N
//                     columns; the accumulator lives in TMEM and each thread folds the heads of its key
//   pg_dsa_topk       the k best keys of every row (radix select; ties go to the earlier position; the list
//                     comes out in position order, so everything downstream is reproducible)
//   pg_dsa_gather     the selected latent rows of every query, copied into pages of their own so that the
//                     dense latent-attention kernel can run over them
//
// Reference parity: pegainfer-kernels/csrc/glm52/{glm52_indexer.cu, glm52_indexer_rope.cu, glm52_deepgemm_mqa.cu,
// glm52_topk.cu} (FP8 MQA logits through DeepGEMM, top-2048); here the logits are bf16 x bf16 -> f32.
#include "common.cuh"

#include <cfloat>

namespace {

// ---------------------------------------------------------------------------------------------
// index key: LayerNorm(weight, bias) -> half-split rotary on the leading `rope` dims -> paged cache
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) dsa_k_append_kernel(const bf16* __restrict__ k, long long ld, const float* __restrict__ nw, const float* __restrict__ nb,
                                                            const bf16* __restrict__ cos, const bf16* __restrict__ sin, const int* __restrict__ positions,
                                                            const int* __restrict__ slots, bf16* __restrict__ cache, int tokens, int d, int rope, int max_pos,
                                                            long long num_slots, float eps, uint32_t* __restrict__ status) {
  PG_PDL_ENTRY();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= tokens) return;
  const int pos = positions[t];
  const long long slot = slots[t];
  if (pos < 0 || pos >= max_pos || slot < 0 || slot >= num_slots) {
    if (lane == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (21u << 8));
    return;
  }
  const bf16* row = k + (long long)t * ld;
  // d <= 256: up to 8 values per lane, element i of the lane is dim lane + 32 * i
  float v[8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < d ? __bfloat162float(row[c]) : 0.f;
    sum += v[i];
  }
  const float mean = warp_sum(sum) / (float)d;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    const float x = c < d ? v[i] - mean : 0.f;
    var += x * x;
  }
  const float inv = rsqrtf(warp_sum(var) / (float)d + eps);
  bf16* out = cache + slot * d;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < d) v[i] = bf16_round((v[i] - mean) * inv * nw[c] + nb[c]);  // the norm's output is a bf16 tensor before the rotation
  }
  // rotation pairs (c, c + rope/2); both live in registers of (possibly) different lanes: go through the cache row
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < d) out[c] = __float2bfloat16(v[i]);
  }
  __syncwarp();
  const int half = rope >> 1;
  for (int c = lane; c < half; c += 32) {
    const float a = __bfloat162float(out[c]), b = __bfloat162float(out[c + half]);
    const float cs = __bfloat162float(cos[(long long)pos * half + c]), sn = __bfloat162float(sin[(long long)pos * half + c]);
    out[c] = __float2bfloat16(a * cs - b * sn);
    out[c + half] = __float2bfloat16(b * cs + a * sn);
  }
}

__global__ void __launch_bounds__(128) dsa_q_rope_kernel(bf16* __restrict__ q, const bf16* __restrict__ cos, const bf16* __restrict__ sin,
                                                          const int* __restrict__ positions, long long units, int heads, int d, int rope, int max_pos) {
  PG_PDL_ENTRY();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long u = (long long)blockIdx.x * 4 + warp;  // (token, head)
  if (u >= units) return;
  const int t = (int)(u / heads);
  const int pos = min(max(positions[t], 0), max_pos - 1);
  bf16* row = q + u * d;
  const int half = rope >> 1;
  for (int c = lane; c < half; c += 32) {
    const float a = __bfloat162float(row[c]), b = __bfloat162float(row[c + half]);
    const float cs = __bfloat162float(cos[(long long)pos * half + c]), sn = __bfloat162float(sin[(long long)pos * half + c]);
    row[c] = __float2bfloat16(a * cs - b * sn);
    row[c + half] = __float2bfloat16(b * cs + a * sn);
  }
}

// ---------------------------------------------------------------------------------------------
// scores on tcgen05: one CTA = (strip of key tiles of 128, query row)
// ---------------------------------------------------------------------------------------------
constexpr int SC_KEYS = 128;
constexpr int SC_D = 128;           // index head dim
constexpr int SC_MAX_HEADS = 64;
struct ScoreSmem {
  uint64_t done;
  uint32_t tmem_slot;
  int abort_flag;
};

constexpr int SC_STRIP = 8;  // key tiles per CTA: set-up (TMEM, barrier, Q staging) once per strip, loads of the next tile under the current one

__global__ void __launch_bounds__(128) dsa_scores_kernel(const bf16* __restrict__ q, const float* __restrict__ w, const bf16* __restrict__ cache,
                                                          const int* __restrict__ unit_seq, const int* __restrict__ q_indptr, const int* __restrict__ kv_lens,
                                                          const int* __restrict__ table, int table_stride, int page_size, long long num_pages, int heads,
                                                          float* __restrict__ scores, int width, uint32_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  // tiles want 1024-byte alignment (128-byte swizzle atoms of 8 rows)
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_tile = tiles;                           // 2 buffers x [2 k-blocks][128 keys][128 B]
  uint8_t* q_tile = tiles + 2 * 2 * SC_KEYS * 128;   // [2 k-blocks][heads][128 B]
  ScoreSmem* sh = reinterpret_cast<ScoreSmem*>(q_tile + 2 * SC_MAX_HEADS * 128);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int t = blockIdx.y, strip = blockIdx.x;
  if (tid == 0) {
    mbar_init(&sh->done, 1);
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  PG_PDL_ENTRY();
  const int b = unit_seq[t];
  const int kv_len = kv_lens[b];
  const int qpos = kv_len - (q_indptr[b + 1] - t);  // rows of a sequence end at its last key
  const int visible = min(kv_len, qpos + 1);        // keys 0 .. visible - 1 may be seen by this row
  const int tile0 = strip * SC_STRIP;
  const int tiles_total = (width + SC_KEYS - 1) / SC_KEYS;
  const int tile_end = min(tile0 + SC_STRIP, tiles_total);
  const int live_tiles = min(tile_end, (visible + SC_KEYS - 1) / SC_KEYS) - tile0;  // tiles of the strip with a visible key
  // tiles wholly in the row's future (or past its sequence): just the fill value
  for (int jt = tile0 + max(live_tiles, 0); jt < tile_end; ++jt)
    if (jt * SC_KEYS + tid < width) scores[(long long)t * width + jt * SC_KEYS + tid] = -INFINITY;
  if (live_tiles <= 0) return;
  if (warp == 0) {
    tmem_alloc(&sh->tmem_slot, 64);
    tmem_relinquish();
  }
  const int* table_row = table + (long long)b * table_stride;
  // this thread's 16 chunks of a key tile: chunk i -> key row (i >> 4), 16-byte column (i & 15), i = tid + 128 n
  auto load_tile = [&](int jt, uint4* regs) {
    const int key0 = jt * SC_KEYS;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const int i = tid + 128 * n, r = i >> 4, c = i & 15;
      const int j = key0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j < visible) {
        const long long page = table_row[j / page_size];
        if (page >= 0 && page < num_pages) v = *reinterpret_cast<const uint4*>(cache + ((page * page_size + j % page_size) * SC_D + c * 8));
        else atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (22u << 8));
      }
      regs[n] = v;
    }
  };
  // 16-byte chunk c of row r lives at chunk (c & 7) ^ (r & 7) of row r in k-block c >> 3 (128-byte swizzle, K-major)
  auto store_tile = [&](uint8_t* dst, const uint4* regs) {
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const int i = tid + 128 * n, r = i >> 4, c = i & 15;
      *reinterpret_cast<uint4*>(dst + (c >> 3) * (SC_KEYS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = regs[n];
    }
  };
  uint4 regs[16];
  load_tile(tile0, regs);
  for (int i = tid; i < heads * 16; i += 128) {
    const int r = i >> 4, c = i & 15;
    const uint4 v = *reinterpret_cast<const uint4*>(q + (((long long)t * heads + r) * SC_D + c * 8));
    *reinterpret_cast<uint4*>(q_tile + (c >> 3) * (SC_MAX_HEADS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
  store_tile(k_tile, regs);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t idesc = umma_idesc_bf16_f32(128, (uint32_t)heads);
  const uint32_t qa = smem_u32(q_tile);
  const float* wt = w + (long long)t * heads;
  bool ok = true;
  for (int lt = 0; lt < live_tiles && ok; ++lt) {
    const int jt = tile0 + lt, buf = lt & 1;
    if (tid == 0) {
      const uint32_t ka = smem_u32(k_tile + buf * (2 * SC_KEYS * 128));
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tmem, umma_desc_k_sw128(ka + kb * (SC_KEYS * 128) + k * 32), umma_desc_k_sw128(qa + kb * (SC_MAX_HEADS * 128) + k * 32), idesc, (kb | k) ? 1u : 0u);
      umma_commit(&sh->done);
    }
    const bool more = lt + 1 < live_tiles;
    if (more) load_tile(jt + 1, regs);  // in flight while the tensor core and the read-back work on this tile
    ok = mbar_wait(&sh->done, (uint32_t)(lt & 1), &sh->abort_flag);
    tc_fence_after();
    if (ok) {
      const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);
      float acc = 0.f;
      for (int c = 0; c < heads; c += 16) {
        uint32_t v[16];
        tmem_ld16(t_row + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc += wt[c + j] * fmaxf(__uint_as_float(v[j]), 0.f);
      }
      const int key = jt * SC_KEYS + tid;
      if (key < width) scores[(long long)t * width + key] = key < visible ? acc : -INFINITY;
    }
    if (more) {
      store_tile(k_tile + (buf ^ 1) * (2 * SC_KEYS * 128), regs);
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();  // the accumulator has been read by every warp and the next tile is staged
    tc_fence_after();
  }
  if (!ok && tid == 0) atomicCAS(status, PG_ST_OK, PG_ST_TIMEOUT | (22u << 8));
  if (warp == 0) tmem_dealloc(tmem, 64);
}

// ---------------------------------------------------------------------------------------------
// top-k per row: radix select, ties to the earlier position, output in position order
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t okey(float f) {  // order-preserving float -> uint
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int TK_THREADS = 1024;

__global__ void __launch_bounds__(TK_THREADS) dsa_topk_kernel(const float* __restrict__ scores, int width, int k, int* __restrict__ out, int* __restrict__ counts) {
  PG_PDL_ENTRY();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_base_sel, s_base_tie;
  __shared__ uint32_t warp_sel[32], warp_tie[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const float* row = scores + (long long)blockIdx.x * width;
  int* dst = out + (long long)blockIdx.x * k;
  const uint32_t NEG_INF = okey(-INFINITY);
  // threshold key: the k-th largest among the finite scores (if there are that many)
  uint32_t prefix = 0, need = (uint32_t)k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += TK_THREADS) hist[i] = 0;
    __syncthreads();
    const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < width; i += TK_THREADS) {
      const uint32_t key = okey(row[i]);
      if (key != NEG_INF && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t n = need, bin = 0;
      bool found = false;
      for (int bq = 255; bq >= 0; --bq) {
        if (hist[bq] >= n) {
          bin = (uint32_t)bq;
          found = true;
          break;
        }
        n -= hist[bq];
      }
      if (!found) {  // fewer finite scores than k: keep them all
        s_prefix = 0;
        s_need = 0xFFFFFFFFu;
      } else {
        s_prefix = prefix | (bin << shift);
        s_need = n;
      }
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    if (need == 0xFFFFFFFFu) break;
    __syncthreads();
  }
  const bool all = need == 0xFFFFFFFFu;  // every finite score is selected
  // ordered compaction: strictly better keys, plus the first `need` keys equal to the threshold
  if (tid == 0) {
    s_base_sel = 0;
    s_base_tie = 0;
  }
  __syncthreads();
  for (int i0 = 0; i0 < width; i0 += TK_THREADS) {
    const int i = i0 + tid;
    uint32_t key = NEG_INF;
    if (i < width) key = okey(row[i]);
    const bool fin = key != NEG_INF;
    const bool tie = fin && !all && key == prefix;
    const unsigned tie_ballot = __ballot_sync(0xFFFFFFFFu, tie);
    const uint32_t tie_before_w = __popc(tie_ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tie[wid] = __popc(tie_ballot);
    __syncthreads();
    uint32_t tie_before = s_base_tie + tie_before_w;
    for (int w2 = 0; w2 < wid; ++w2) tie_before += warp_tie[w2];
    const bool sel = fin && (all || key > prefix || (tie && tie_before < need));
    const unsigned sel_ballot = __ballot_sync(0xFFFFFFFFu, sel);
    const uint32_t sel_before_w = __popc(sel_ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_sel[wid] = __popc(sel_ballot);
    __syncthreads();
    uint32_t at = s_base_sel + sel_before_w;
    for (int w2 = 0; w2 < wid; ++w2) at += warp_sel[w2];
    if (sel && at < (uint32_t)k) dst[at] = i;
    __syncthreads();
    if (tid == 0) {
      uint32_t a = 0, c = 0;
      for (int w2 = 0; w2 < TK_THREADS / 32; ++w2) {
        a += warp_sel[w2];
        c += warp_tie[w2];
      }
      s_base_sel += a;
      s_base_tie += c;
    }
    __syncthreads();
  }
  const uint32_t total = min(s_base_sel, (uint32_t)k);
  for (int i = (int)total + tid; i < k; i += TK_THREADS) dst[i] = -1;
  if (tid == 0) counts[blockIdx.x] = (int)total;
}

// ---------------------------------------------------------------------------------------------
// gather the selected latent rows of each query into pages of a scratch cache
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) dsa_gather_kernel(const bf16* __restrict__ latent, const int* __restrict__ select, int k, const int* __restrict__ unit_seq,
                                                          const int* __restrict__ table, int table_stride, int page_size, long long num_pages, int row_words,
                                                          uint4* __restrict__ out, int slots_per_row, uint32_t* __restrict__ status) {
  PG_PDL_ENTRY();
  const int t = blockIdx.y;
  const int b = unit_seq[t];
  const int chunks = row_words;  // 16-byte chunks per latent row
  for (int e = blockIdx.x * 4 + (threadIdx.x >> 5); e < k; e += gridDim.x * 4) {
    const int j = select[(long long)t * k + e];
    if (j < 0) continue;
    const long long page = table[(long long)b * table_stride + j / page_size];
    if (page < 0 || page >= num_pages) {
      if ((threadIdx.x & 31) == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (23u << 8));
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(latent) + (page * page_size + j % page_size) * chunks;
    uint4* dst = out + ((long long)t * slots_per_row + e) * chunks;
    for (int c = threadIdx.x & 31; c < chunks; c += 32) dst[c] = src[c];
  }
}

}  // namespace

extern "C" int pg_dsa_k_append(const void* k, long long ld, const void* norm_w, const void* norm_b, const void* cos, const void* sin, const void* positions,
                               const void* slots, void* cache, int tokens, int d, int rope, int max_pos, long long num_slots, float eps, void* status,
                               cudaStream_t stream) {
  PG_REQUIRE(d <= 256 && rope % 2 == 0 && rope <= d, "dsa_k_append: head dim %d / rope %d not supported", d, rope);
  if (tokens == 0) return PG_OK;
  PG_CUDA(launch_pdl(dsa_k_append_kernel, dim3((tokens + 3) / 4), dim3(128), (size_t)0, stream, (const bf16*)k, ld, (const float*)norm_w, (const float*)norm_b,
                     (const bf16*)cos, (const bf16*)sin, (const int*)positions, (const int*)slots, (bf16*)cache, tokens, d, rope, max_pos, num_slots, eps,
                     (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_dsa_q_rope(void* q, const void* cos, const void* sin, const void* positions, int tokens, int heads, int d, int rope, int max_pos,
                             cudaStream_t stream) {
  PG_REQUIRE(rope % 2 == 0 && rope <= d, "dsa_q_rope: head dim %d / rope %d not supported", d, rope);
  const long long units = (long long)tokens * heads;
  if (units == 0) return PG_OK;
  PG_CUDA(launch_pdl(dsa_q_rope_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), (size_t)0, stream, (bf16*)q, (const bf16*)cos, (const bf16*)sin,
                     (const int*)positions, units, heads, d, rope, max_pos));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_dsa_scores(const void* q, const void* w, const void* cache, const void* unit_seq, const void* q_indptr, const void* kv_lens, const void* table,
                             int table_stride, int page_size, long long num_pages, int tokens, int heads, int d, void* scores, int width, void* status,
                             cudaStream_t stream) {
  PG_REQUIRE(d == SC_D, "dsa_scores: built for an index head dim of 128 (got %d)", d);
  PG_REQUIRE(heads % 16 == 0 && heads >= 16 && heads <= SC_MAX_HEADS, "dsa_scores: %d index heads (need a multiple of 16 up to 64)", heads);
  if (tokens == 0 || width == 0) return PG_OK;
  const size_t smem = 1024 + 2 * 2 * SC_KEYS * 128 + 2 * SC_MAX_HEADS * 128 + sizeof(ScoreSmem);
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(dsa_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(dsa_scores_kernel, dim3((unsigned)ceil_div(ceil_div(width, SC_KEYS), SC_STRIP), (unsigned)tokens), dim3(128), smem, stream, (const bf16*)q, (const float*)w,
                     (const bf16*)cache, (const int*)unit_seq, (const int*)q_indptr, (const int*)kv_lens, (const int*)table, table_stride, page_size, num_pages,
                     heads, (float*)scores, width, (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_dsa_topk(const void* scores, int rows, int width, int k, void* out, void* counts, cudaStream_t stream) {
  if (rows == 0) return PG_OK;
  PG_REQUIRE(k > 0, "dsa_topk: k must be positive");
  PG_CUDA(launch_pdl(dsa_topk_kernel, dim3((unsigned)rows), dim3(TK_THREADS), (size_t)0, stream, (const float*)scores, width, k, (int*)out, (int*)counts));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

extern "C" int pg_dsa_gather(const void* latent, const void* select, int k, const void* unit_seq, const void* table, int table_stride, int page_size,
                             long long num_pages, int row_bytes, int rows, void* out, int slots_per_row, void* status, cudaStream_t stream) {
  PG_REQUIRE(row_bytes % 16 == 0, "dsa_gather: latent rows of %d bytes are not a multiple of 16", row_bytes);
  if (rows == 0) return PG_OK;
  PG_CUDA(launch_pdl(dsa_gather_kernel, dim3((unsigned)min(ceil_div(k, 4), 64), (unsigned)rows), dim3(128), (size_t)0, stream, (const bf16*)latent,
                     (const int*)select, k, (const int*)unit_seq, (const int*)table, table_stride, page_size, num_pages, row_bytes / 16, (uint4*)out, slots_per_row,
                     (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
