// Causal GQA attention over the paged KV cache for wide heads (head dim 512: the global layers of the Gemma 4 line),
// prefill chunks and decode rows alike.
//
// One block per (query row, KV head): its warps are the query heads that share the KV head, so a tile of keys and values
// is fetched through the page table once and used by all of them from shared memory.  A lane holds D / 32 consecutive
// elements of its head's query row and of the output row; per tile of 16 keys a warp computes the 16 scores (dot
// products reduced over the warp), one running-maximum update, and the weighted sum of the 16 value rows.  Plain CUDA
// cores: these layers are one in six of the model, and head dim 512 leaves no room in tensor memory for the accumulators
// of the tcgen05 kernels (O alone would take all 512 columns).
//
// Reference parity: pegainfer-kernels/csrc/shared/prefill_attention_hd512.cu:64-540, paged_attention_hd512.cu:71-224.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int TK = 16;  // keys per tile

struct WideParams {
  const bf16* q;        // [T, hq, D]
  const bf16* kv;       // [pages, 2, page_size, hkv, D]
  bf16* out;            // [T, hq * D]
  const int* unit_seq;  // [T] sequence of every query row
  const int* q_indptr;  // [num_seqs + 1]
  const int* kv_lens;   // [num_seqs]
  const int* table;     // [num_seqs, table_stride]
  int table_stride, tokens, hq, hkv, page_size, window;
  long long num_pages;
  float scale;
  uint32_t* status;
};

template <int D>
__global__ void __launch_bounds__(256) attn_wide_kernel(const WideParams p) {
  PG_PDL_ENTRY();
  constexpr int E = D / 32;  // elements per lane
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* k_tile = reinterpret_cast<bf16*>(smem_raw);  // [TK][D]
  bf16* v_tile = k_tile + TK * D;                    // [TK][D]
  const int t = blockIdx.x, hk = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.hq / p.hkv;
  const int head = hk * group + warp;
  const int b = p.unit_seq[t];
  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int pos = kv_len - q_len + (t - q0);  // position of this query row
  bf16* dst = p.out + ((long long)t * p.hq + head) * D + lane * E;
  if (kv_len <= 0 || pos < 0) {  // padding rows of a graph bucket attend to nothing
#pragma unroll
    for (int e = 0; e < E; e += 8) *reinterpret_cast<uint4*>(dst + e) = make_uint4(0, 0, 0, 0);
    return;
  }
  const int start = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int* table_row = p.table + (long long)b * p.table_stride;

  float q[E], o[E];
  {
    const bf16* src = p.q + ((long long)t * p.hq + head) * D + lane * E;
#pragma unroll
    for (int e = 0; e < E; e += 8) {
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(src + e), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) q[e + i] = f[i] * p.scale;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  for (int tile0 = start / TK * TK; tile0 <= pos; tile0 += TK) {
    __syncthreads();  // the previous tile has been consumed by every warp
    for (int idx = threadIdx.x; idx < 2 * TK * CHUNKS; idx += blockDim.x) {
      const int which = idx / (TK * CHUNKS), rem = idx % (TK * CHUNKS);
      const int j = rem / CHUNKS, c = rem % CHUNKS;
      const int tok = tile0 + j;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (tok <= pos && tok >= start) {
        int page = table_row[tok / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (46u << 8));
          page = 0;
        }
        val = *reinterpret_cast<const uint4*>(p.kv + ((((long long)page * 2 + which) * p.page_size + tok % p.page_size) * p.hkv + hk) * D + c * 8);
      }
      *reinterpret_cast<uint4*>((which ? v_tile : k_tile) + j * D + c * 8) = val;
    }
    __syncthreads();
    float s[TK];
    float tile_max = -INFINITY;
#pragma unroll
    for (int j = 0; j < TK; ++j) {
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < E; e += 8) {
        float f[8];
        unpack8(*reinterpret_cast<const bf16x8*>(k_tile + j * D + lane * E + e), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(q[e + i], f[i], acc);
      }
      acc = warp_sum(acc);
      const int tok = tile0 + j;
      s[j] = (tok <= pos && tok >= start) ? acc : -INFINITY;
      tile_max = fmaxf(tile_max, s[j]);
    }
    if (tile_max == -INFINITY) continue;  // uniform across the block's warps: depends on positions only
    const float m_new = fmaxf(m, tile_max);
    const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
    l *= corr;
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] *= corr;
#pragma unroll
    for (int j = 0; j < TK; ++j) {
      const float pj = s[j] == -INFINITY ? 0.f : __expf(s[j] - m_new);
      l += pj;
#pragma unroll
      for (int e = 0; e < E; e += 8) {
        float f[8];
        unpack8(*reinterpret_cast<const bf16x8*>(v_tile + j * D + lane * E + e), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[e + i] = fmaf(pj, f[i], o[e + i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int e = 0; e < E; e += 8) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = o[e + i] * inv;
    *reinterpret_cast<bf16x8*>(dst + e) = pack8(f);
  }
}

}  // namespace

// q [T, hq, dim] bf16, kv_layer [pages, 2, page_size, hkv, dim], out [T, hq * dim]; `unit_seq[t]` = sequence of row t.
extern "C" int pg_attention_wide(const void* q, const void* kv_layer, void* out, const void* unit_seq, const void* q_indptr, const void* kv_lens, const void* table,
                                 int table_stride, int tokens, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int window, void* status,
                                 cudaStream_t stream) {
  PG_REQUIRE(dim == 512, "wide attention is built for head dim 512 (got %d)", dim);
  PG_REQUIRE(hq % hkv == 0 && hq / hkv >= 1 && hq / hkv <= 8, "wide attention: %d query heads per KV head (1 .. 8)", hkv ? hq / hkv : 0);
  if (tokens == 0) return PG_OK;
  WideParams p;
  p.q = (const bf16*)q;
  p.kv = (const bf16*)kv_layer;
  p.out = (bf16*)out;
  p.unit_seq = (const int*)unit_seq;
  p.q_indptr = (const int*)q_indptr;
  p.kv_lens = (const int*)kv_lens;
  p.table = (const int*)table;
  p.table_stride = table_stride;
  p.tokens = tokens;
  p.hq = hq;
  p.hkv = hkv;
  p.page_size = page_size;
  p.window = window;
  p.num_pages = num_pages;
  p.scale = scale;
  p.status = (uint32_t*)status;
  const size_t smem = 2 * (size_t)TK * 512 * 2;
  PG_CUDA(launch_pdl(attn_wide_kernel<512>, dim3((unsigned)tokens, (unsigned)hkv), dim3((unsigned)(32 * (hq / hkv))), smem, stream, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
