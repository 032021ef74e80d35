// Causal GQA attention over the paged KV cache for wide heads (head dim 512: the global layers of the Gemma 4 line),
// prefill chunks and decode rows alike.  Head dim 512 leaves no room in tensor memory for the accumulators of the tcgen05
// kernels (O alone would take all 512 columns), so this head dim runs on `mma.sync` with the head split over the warps
// of a block (second kernel below); the first kernel is the plain CUDA-core form, kept for query-head groups that do not
// divide 16 and as the oracle-like fallback (`PEGAINFER_WIDE_MMA=0`).
//
// CUDA-core kernel: one block per (query row, KV head): its warps are the query heads that share the KV head, so a tile
// of keys and values is fetched through the page table once and used by all of them from shared memory.  A lane holds
// D / 32 consecutive elements of its head's query row and of the output row; per tile of 16 keys a warp computes the 16
// scores (dot products reduced over the warp), one running-maximum update, and the weighted sum of the 16 value rows.
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
  // split KV (decode steps of few long sequences): split s of a block's key tiles writes its unnormalised O and (m, l)
  // per row; attn_wide_merge_kernel combines them
  int splits;
  float* part_o;   // [T * hq, splits, D]
  float* part_ml;  // [T * hq, splits, 2]
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

// ---------------------------------------------------------------------------------------------------------------------
// Tensor-core variant (mma.sync m16n8k16, bf16 in, f32 accumulate).  A block of eight warps owns two MMA row tiles of 16
// rows: 32 / G consecutive query tokens of a sequence times the G query heads of one KV head, so prefill chunks and
// decode rows alike fetch a key / value tile once for the whole group.  The head dim is split over the four warps of a
// row tile: warp w multiplies Q[:, 128 w : 128 w + 128] with the same slice of the 32 keys of a tile, the four partial
// score tiles are summed through shared memory, every warp runs the (identical) online softmax, and accumulates its own
// 128 columns of O.  K / V tiles of 32 keys x 512 are double-buffered by cp.async through the page table.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Swizzled offset (in bf16 elements) of 16-byte chunk `ch` of row `r` in a [rows][D] tile.
template <int D>
__device__ __forceinline__ int swz(int r, int ch) {
  return r * D + ((ch ^ (r & 7)) << 3);
}

constexpr float NEG_BIG = -1e30f;

constexpr int WIDE_ROWS = 32;  // query rows (tokens x heads of the group) per block: two MMA row tiles

template <int D>
__global__ void __launch_bounds__(256, 1) attn_wide_mma_kernel(const WideParams p, int num_seqs) {
  PG_PDL_ENTRY();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int BKV = 32;
  constexpr int CH = D / 8;    // 16-byte chunks per row
  constexpr int SL = D / 4;    // columns of one warp's slice (128)
  constexpr int KS = SL / 16;  // k-steps of the slice in Q K^T
  constexpr int NT = SL / 8;   // n-tiles of the slice in P V
  constexpr int TILE_ELEMS = BKV * D;
  bf16* sm = reinterpret_cast<bf16*>(smem_raw);                             // [2 stages][K | V][32][D]; the Q tile is staged in stage 0 first
  float* s_part = reinterpret_cast<float*>(sm + 2 * 2 * TILE_ELEMS);        // [8 warps][BKV / 8][32 lanes][4]
  const int warp_id = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt = warp_id >> 2, warp = warp_id & 3;  // row tile of 16 rows, slice of the head dim
  const int g = lane >> 2, t4 = lane & 3;
  const int hk = blockIdx.y;
  const int G = p.hq / p.hkv;
  const int TPT = WIDE_ROWS / G;  // query tokens per block

  int b = 0, tile_in_seq = 0;
  {
    int rem = (int)(gridDim.x / (unsigned)p.splits) - 1 - (int)(blockIdx.x / (unsigned)p.splits);  // late tiles (most keys) first
    for (; b < num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + TPT - 1) / TPT;
      if (rem < nt) {
        tile_in_seq = rem;
        break;
      }
      rem -= nt;
    }
    if (b >= num_seqs) return;
  }
  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int* table_row = p.table + (long long)b * p.table_stride;
  const int tok_base_q = tile_in_seq * TPT;  // first query token of this tile within the sequence
  const int toks_here = min(TPT, q_len - tok_base_q);
  const int pos_base = kv_len - q_len + tok_base_q;
  if (kv_len <= 0 || pos_base + toks_here - 1 < 0) {  // padding rows of a graph bucket attend to nothing
    if (p.splits > 1) {  // the merge kernel writes the zeros: every split reports an empty partial
      for (int r = threadIdx.x; r < toks_here * G; r += 256) {
        const long long row = (long long)(q0 + tok_base_q + r / G) * p.hq + hk * G + r % G;
        p.part_ml[(row * p.splits + (int)(blockIdx.x % (unsigned)p.splits)) * 2] = NEG_BIG;
        p.part_ml[(row * p.splits + (int)(blockIdx.x % (unsigned)p.splits)) * 2 + 1] = 0.f;
      }
      return;
    }
    for (int idx = threadIdx.x; idx < toks_here * G * CH; idx += 256) {
      const int r = idx / CH, ch = idx % CH;
      *reinterpret_cast<uint4*>(p.out + ((long long)(q0 + tok_base_q + r / G) * p.hq + hk * G + r % G) * D + ch * 8) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  // stage the Q tile [32][D] (row r = token r / G, head hk G + r % G), then the warp's A fragments of its slice
  for (int c = threadIdx.x; c < WIDE_ROWS * CH; c += 256) {
    const int r = c / CH, ch = c % CH;
    const bool valid = r / G < toks_here;
    const bf16* src = p.q + ((long long)(q0 + tok_base_q + (valid ? r / G : 0)) * p.hq + hk * G + r % G) * D + ch * 8;
    cp_async16(sm + swz<D>(r, ch), src, valid);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int j = lane >> 3, r = lane & 7;
    const int row = rt * 16 + (j & 1) * 8 + r;
    const int ch = warp * (SL / 8) + ks * 2 + (j >> 1);
    ldsm_x4(smem_u32(sm + swz<D>(row, ch)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }
  __syncthreads();

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};
  const bool rt_active = (rt * 16) / G < toks_here;

  const int max_pos = pos_base + toks_here - 1;
  int kv_start = 0;
  if (p.window > 0) kv_start = max(0, pos_base - p.window + 1) / BKV * BKV;
  const int kv_end = min(kv_len, max_pos + 1);
  const int split = (int)(blockIdx.x % (unsigned)p.splits);
  const int all_tiles = (kv_end - kv_start + BKV - 1) / BKV;
  const int tps = (all_tiles + p.splits - 1) / p.splits;  // key tiles per split
  kv_start += split * tps * BKV;
  const int n_kv_tiles = max(0, min(tps, all_tiles - split * tps));

  constexpr int RPT = BKV * CH / 256, RSTEP = 256 / CH;
  const long long row_stride = (long long)p.hkv * D;
  const long long v_plane = (long long)p.page_size * row_stride;
  const int my_ch = threadIdx.x % CH, my_r0 = threadIdx.x / CH;
  const bf16* kv_head = p.kv + (long long)hk * D + my_ch * 8;
  auto issue = [&](int kt, int stage) {
    bf16* ks_ = sm + stage * 2 * TILE_ELEMS;
    bf16* vs_ = ks_ + TILE_ELEMS;
    if (kt < n_kv_tiles) {
      const int tok_base = kv_start + kt * BKV;
#pragma unroll 4
      for (int i = 0; i < RPT; ++i) {
        const int r = my_r0 + i * RSTEP;
        const bool valid = tok_base + r < kv_end;
        const int tok = valid ? tok_base + r : kv_start;
        int page = table_row[tok / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (47u << 8));
          page = 0;
        }
        const bf16* src = kv_head + ((long long)page * 2 * p.page_size + tok % p.page_size) * row_stride;
        cp_async16(ks_ + swz<D>(r, my_ch), src, valid);
        cp_async16(vs_ + swz<D>(r, my_ch), src + v_plane, valid);
      }
    }
    cp_async_commit();
  };

  issue(0, 0);
  const float scale_log2 = p.scale * 1.4426950408889634f;
  for (int kt = 0; kt < n_kv_tiles; ++kt) {
    issue(kt + 1, (kt + 1) & 1);
    cp_async_wait<1>();
    __syncthreads();
    const bf16* ks_ = sm + (kt & 1) * 2 * TILE_ELEMS;
    const bf16* vs_ = ks_ + TILE_ELEMS;
    const int tok_base = kv_start + kt * BKV;
    float s_acc[BKV / 8][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
    // a row tile without live rows (decode: one token per sequence fills at most the first tile) only copies and waits
    if (rt_active) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < BKV / 16; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = n2 * 16 + (j >> 1) * 8 + r;
        const int ch = warp * (SL / 8) + ks * 2 + (j & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(ks_ + swz<D>(row, ch)), b0, b1, b2, b3);
        mma16816(s_acc[2 * n2], qf[ks], b0, b1);
        mma16816(s_acc[2 * n2 + 1], qf[ks], b2, b3);
      }
    }
    // sum the four warps' partial scores (each over its 128 columns of the head)
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n)
      *reinterpret_cast<float4*>(s_part + ((warp_id * (BKV / 8) + n) * 32 + lane) * 4) = make_float4(s_acc[n][0], s_acc[n][1], s_acc[n][2], s_acc[n][3]);
    }
    __syncthreads();
    if (rt_active) {
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(s_part + (((rt * 4 + w) * (BKV / 8) + n) * 32 + lane) * 4);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      s_acc[n][0] = acc.x;
      s_acc[n][1] = acc.y;
      s_acc[n][2] = acc.z;
      s_acc[n][3] = acc.w;
    }
    float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok_base + n * 8 + 2 * t4 + (e & 1);
        const int tq = (rt * 16 + g + (e >> 1) * 8) / G;
        const int qp = pos_base + tq;
        bool ok = tq < toks_here && tok <= qp && tok < kv_end;
        if (p.window > 0) ok = ok && tok > qp - p.window;
        const float v = ok ? s_acc[n][e] * scale_log2 : NEG_BIG;
        s_acc[n][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float m_new = fmaxf(m_run[rr], mx[rr]);
      corr[rr] = exp2f(m_run[rr] - m_new);
      m_run[rr] = m_new;
    }
    float ps[2] = {0.f, 0.f};
    uint32_t pa[BKV / 16][4];
#pragma unroll
    for (int n = 0; n < BKV / 8; ++n) {
      float pvv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pvv[e] = s_acc[n][e] <= NEG_BIG ? 0.f : exp2f(s_acc[n][e] - m_run[e >> 1]);
        ps[e >> 1] += pvv[e];
      }
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(pvv[0], pvv[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(pvv[2], pvv[3]);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 1);
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 2);
      l_run[rr] = l_run[rr] * corr[rr] + ps[rr];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        const int j = lane >> 3, r = lane & 7;
        const int row = kk * 16 + (j & 1) * 8 + r;
        const int ch = warp * (SL / 8) + n2 * 2 + (j >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vs_ + swz<D>(row, ch)), b0, b1, b2, b3);
        mma16816(o[2 * n2], pa[kk], b0, b1);
        mma16816(o[2 * n2 + 1], pa[kk], b2, b3);
      }
    }
    }
    __syncthreads();  // the tile and the partial-score buffer are free again
  }
  cp_async_wait<0>();

#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = rt * 16 + g + rr * 8;
    const int tq = r / G;
    if (tq < toks_here) {
      const long long row = (long long)(q0 + tok_base_q + tq) * p.hq + hk * G + r % G;
      if (p.splits > 1) {  // unnormalised partial of this split and its (running maximum in the log2 domain, sum)
        float* po = p.part_o + (row * p.splits + split) * D + warp * SL;
#pragma unroll
        for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(po + n * 8 + 2 * t4) = make_float2(o[n][rr * 2], o[n][rr * 2 + 1]);
        if (warp == 0 && t4 == 0) {
          p.part_ml[(row * p.splits + split) * 2] = m_run[rr];
          p.part_ml[(row * p.splits + split) * 2 + 1] = l_run[rr];
        }
        continue;
      }
      const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
      bf16* dst = p.out + row * D + warp * SL;
#pragma unroll
      for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
    }
  }
}

// One warp per output row: combine the splits' partials.
template <int D>
__global__ void __launch_bounds__(128) attn_wide_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out, long long rows, int splits) {
  PG_PDL_ENTRY();
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = NEG_BIG;
  for (int s2 = 0; s2 < splits; ++s2) mx = fmaxf(mx, part_ml[(row * splits + s2) * 2]);
  float l = 0.f;
  constexpr int E = D / 32;
  float acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  for (int s2 = 0; s2 < splits; ++s2) {
    const float m = part_ml[(row * splits + s2) * 2], ls = part_ml[(row * splits + s2) * 2 + 1];
    if (ls <= 0.f) continue;
    const float w = exp2f(m - mx);
    l += w * ls;
    const float* po = part_o + (row * splits + s2) * D + lane * E;
#pragma unroll
    for (int e = 0; e < E; e += 4) {
      const float4 v = *reinterpret_cast<const float4*>(po + e);
      acc[e] += w * v.x;
      acc[e + 1] += w * v.y;
      acc[e + 2] += w * v.z;
      acc[e + 3] += w * v.w;
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  bf16* dst = out + row * D + lane * E;
#pragma unroll
  for (int e = 0; e < E; e += 8) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = acc[e + i] * inv;
    *reinterpret_cast<bf16x8*>(dst + e) = pack8(f);
  }
}

}  // namespace

// q [T, hq, dim] bf16, kv_layer [pages, 2, page_size, hkv, dim], out [T, hq * dim]; `unit_seq[t]` = sequence of row t.
// `q_tiles` = sum over the sequences of ceil(query rows / (32 / (hq / hkv))) selects the tensor-core kernel (hq / hkv a
// divisor of 32); 0 selects the CUDA-core kernel.
extern "C" int pg_attention_wide(const void* q, const void* kv_layer, void* out, const void* unit_seq, const void* q_indptr, const void* kv_lens, const void* table,
                                 int table_stride, int tokens, int num_seqs, int q_tiles, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int window,
                                 int splits, void* part_o, void* part_ml, void* status, cudaStream_t stream) {
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
  p.splits = splits < 1 ? 1 : splits;
  p.part_o = (float*)part_o;
  p.part_ml = (float*)part_ml;
  PG_REQUIRE(p.splits == 1 || (part_o && part_ml && q_tiles > 0), "wide attention: split KV needs the partial buffers and the tensor-core kernel");
  const int group = hq / hkv;
  if (q_tiles > 0 && WIDE_ROWS % group == 0) {
    const size_t smem_mma = (size_t)2 * 2 * 32 * 512 * 2 + (size_t)8 * 4 * 32 * 4 * 4;
    static bool attr_done = false;
    if (!attr_done) {
      PG_CUDA(cudaFuncSetAttribute(attn_wide_mma_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma));
      attr_done = true;
    }
    PG_CUDA(launch_pdl(attn_wide_mma_kernel<512>, dim3((unsigned)(q_tiles * p.splits), (unsigned)hkv), dim3(256), smem_mma, stream, p, num_seqs));
    PG_LAUNCH_CHECK();
    if (p.splits > 1) {
      const long long rows = (long long)tokens * hq;
      PG_CUDA(launch_pdl(attn_wide_merge_kernel<512>, dim3((unsigned)((rows + 3) / 4)), dim3(128), (size_t)0, stream, (const float*)p.part_o, (const float*)p.part_ml, p.out, rows, p.splits));
      PG_LAUNCH_CHECK();
    }
    return PG_OK;
  }
  const size_t smem = 2 * (size_t)TK * 512 * 2;
  PG_CUDA(launch_pdl(attn_wide_kernel<512>, dim3((unsigned)tokens, (unsigned)hkv), dim3((unsigned)(32 * (hq / hkv))), smem, stream, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
