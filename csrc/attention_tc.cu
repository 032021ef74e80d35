// Prefill attention on tcgen05 for sm_100a: causal GQA attention of ragged query rows over a paged KV cache,
// head dims 128 and 256 (the second kernel, further down, has its own notes).
//
// Head dim 128: one CTA owns 256 query rows of one query head as two tiles of 128 (two softmax groups) and walks the KV
// of its sequence in tiles of 128 keys that both tiles share:
//
//   S_g = Q_g K^T      tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), accumulator in TMEM
//   P_g = softmax tile four warps per group, one query row per thread: the row of S is read into registers in one round
//                      trip (maximum with three-input max, exponentials with packed f32x2 arithmetic and ex2.approx),
//                      P is written back as bf16 INTO TENSOR MEMORY over the first score columns (two values per 32-bit
//                      column).  Whether a tile needs the causal / length mask is a compile-time property of the tile
//                      body: the plain tiles carry no compare or select per element.
//   O_g += P_g V       tcgen05.mma with A = P_g read from tensor memory and V as an MN-major B operand (the cache stores
//                      keys as rows, which is what the contraction over keys needs transposed); O_g stays in TMEM for
//                      the whole walk.  It is rescaled (tcgen05.ld / multiply / tcgen05.st) only when a row's maximum
//                      grew by more than 2^8 since the value its exponentials refer to; the row sum follows the same
//                      reference, so the result is exact.
//
// Roles: warp 0 = TMA producer (Q once, then K and V tiles through the page table, two stages each; a tile is 4 x pages
// small boxes, which the 32 lanes issue side by side, with the page ids read one tile ahead), warp 1 = MMA issuer, in the
// order  P V of group a, next S of group a, P V of group b, next S of group b : while one group's softmax runs the
// tensor core has the other group's work, warps 2-5 / 6-9 = softmax groups a / b and output.
// TMEM: S / P of group g at columns 128 g, O of group g at 256 + 128 g.  The grid is one-dimensional with the query
// tile slowest and late tiles first, so the CTAs with the most keys start first on every SM.  Every wait is bounded and
// reports through the status word.
//
// Reference parity: the reference's prefill attention is FlashInfer's BatchPrefillWithPagedKVCache
// (pegainfer-kernels/csrc/shared/flashinfer_prefill.cu, hd256 instantiations in paged_attention.cu:977-1135), an
// mma.sync kernel on every architecture.
#include <type_traits>
#include "common.cuh"

#include <cuda.h>

#include <mutex>

namespace {

constexpr int BQ2 = 256, BKV = 128, D = 128;
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
  int window;             // head dim 256 only: a row sees its last `window` keys (0: all of them)
  int mn_lbo_first;       // descriptor variant of the MN-major operand (1: LBO = stride between 64-column blocks)
  uint32_t* status;
};

constexpr int GROUPS = 2;          // query tiles of 128 rows per CTA; their softmax groups alternate on the tensor core
constexpr int THREADS = 64 + GROUPS * 128;
constexpr float RESCALE_LOG2 = 8.f;  // O and the row sum move to a new maximum only when it grew by more than 2^8

struct TcSmem {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[GROUPS], p_ready[GROUPS], o_full[GROUPS];
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
// Each thread of the warp writes 16 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: A is a 128-row matrix in tensor memory (row = lane, two bf16 per 32-bit column).
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(THREADS, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* q_tile = tiles;                            // GROUPS x 32 KB
  uint8_t* k_tile = tiles + GROUPS * TILE_BYTES;      // 2 x 32 KB
  uint8_t* v_tile = k_tile + 2 * TILE_BYTES;          // 2 x 32 KB
  TcSmem* sh = reinterpret_cast<TcSmem*>(v_tile + 2 * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, query tile slowest: every head's late tiles (most keys) are handed out before any early
  // tile, so the long CTAs start first on all SMs and the short ones fill the tail
  const int hq = (int)(blockIdx.x % (unsigned)p.hq);
  const int h = hq / (p.hq / p.hkv);

  // (sequence, query tile of 256 rows) of this CTA: late tiles (most keys) first
  int b = 0, tile_in_seq = 0;
  {
    int rem = (int)(gridDim.x / (unsigned)p.hq) - 1 - (int)(blockIdx.x / (unsigned)p.hq);
    for (; b < p.num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + BQ2 - 1) / BQ2;
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
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(&sh->k_full[s2], 1);
      mbar_init(&sh->k_empty[s2], 1);
      mbar_init(&sh->v_full[s2], 1);
      mbar_init(&sh->v_empty[s2], 1);
    }
    for (int g = 0; g < GROUPS; ++g) {
      mbar_init(&sh->s_full[g], 1);
      mbar_init(&sh->p_ready[g], 4);
      mbar_init(&sh->o_full[g], 1);
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
  const uint32_t tmem = sh->tmem_slot;  // columns: S of group g at 128 g (P overwrites its first 64), O of group g at 256 + 128 g
  volatile int* abort_flag = &sh->abort_flag;
  PG_PDL_ENTRY();

  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int row_base = tile_in_seq * BQ2;
  const int rows_here = min(BQ2, q_len - row_base);
  const int pos_base = kv_len - q_len + row_base;  // position of the CTA's first row
  // tiles of 128 keys each group needs: up to its last row's position
  int n_g[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int rows_of_g = min(128, rows_here - g * 128);
    n_g[g] = (rows_of_g > 0 && kv_len > 0) ? min(pos_base + g * 128 + rows_of_g - 1, kv_len - 1) / BKV + 1 : 0;
  }
  const int n_tiles = max(n_g[0], n_g[1]);
  const int* table_row = p.table + (long long)b * p.table_stride;

  if (warp == 0) {
    // Producer warp.  A key tile and its value tile arrive as 4 * ppt small boxes (one per page, 64-column half and
    // K or V); the lanes issue them side by side, slot = lane, lane + 32, and each lane reads the page ids of its own
    // slots one tile ahead, so that neither the table's memory latency nor a serial run of TMA issues sits between
    // two tiles.
    if (n_tiles > 0) {
      const uint64_t pol = l2_policy_evict_normal();
      if (lane == 0) {
        mbar_expect_tx(&sh->q_full, GROUPS * TILE_BYTES);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          tma_load_3d(q_tile + g * TILE_BYTES, &tm_q, &sh->q_full, 0, hq, q0 + row_base + g * 128, pol);
          tma_load_3d(q_tile + g * TILE_BYTES + HALF_BYTES, &tm_q, &sh->q_full, 64, hq, q0 + row_base + g * 128, pol);
        }
      }
      const int ppt = BKV / p.page_size;  // pages per key tile (1 .. 16)
      const int per_kv = 2 * ppt, slots = 4 * ppt;
      auto page_of = [&](int j, int slot) -> int {
        const int pg = (slot % per_kv) >> 1;
        const int pages_live = min(ppt, (kv_len - j * BKV + p.page_size - 1) / p.page_size);
        int page = (slot < slots && pg < pages_live) ? __ldg(table_row + j * ppt + pg) : 0;  // past the end: the padding page, keys masked
        if (page < 0 || page >= p.num_pages) {
          atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (41u << 8));
          page = 0;
        }
        return page;
      };
      int nxt0 = page_of(0, lane), nxt1 = page_of(0, lane + 32);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int pg0 = nxt0, pg1 = nxt1;
        if (j + 1 < n_tiles) {
          nxt0 = page_of(j + 1, lane);
          nxt1 = page_of(j + 1, lane + 32);
        }
        const int st = j & 1;
        if (j >= 2) {
          const uint32_t par = (uint32_t)(((j >> 1) - 1) & 1);
          ok = mbar_wait(&sh->k_empty[st], par, abort_flag) && mbar_wait(&sh->v_empty[st], par, abort_flag);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
        }
        if (lane == 0) {
          mbar_expect_tx(&sh->k_full[st], TILE_BYTES);
          mbar_expect_tx(&sh->v_full[st], TILE_BYTES);
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int slot = lane + 32 * it;
          if (slot < slots) {
            const int kvsel = slot / per_kv, rem = slot % per_kv, pg = rem >> 1, half = rem & 1;
            const int z = ((it ? pg1 : pg0) * 2 + kvsel) * p.page_size;
            uint8_t* dst = (kvsel ? v_tile : k_tile) + st * TILE_BYTES + half * HALF_BYTES + pg * p.page_size * 128;
            tma_load_3d(dst, &tm_kv, kvsel ? &sh->v_full[st] : &sh->k_full[st], half * 64, h, z, pol);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_o = idesc_bf16(128, 128, 1);
      const uint32_t lbo = p.mn_lbo_first ? (uint32_t)HALF_BYTES : 1024u, sbo = p.mn_lbo_first ? 1024u : (uint32_t)HALF_BYTES;
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      int k_seen = -1, v_seen = -1;  // tiles whose K / V arrival this thread has already observed
      // S of group g, tile j.  K_j is released once the last group that needs it has issued its S.  S of tile j
      // overwrites the group's previous S and P: the tensor core runs this thread's instructions in order, and the
      // product that read that P was issued before.
      auto issue_s = [&](int g, int j) {
        if (j >= n_g[g]) return true;
        const int st = j & 1;
        if (k_seen < j) {
          if (!mbar_wait(&sh->k_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
          k_seen = j;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(q_tile + g * TILE_BYTES), ka = smem_u32(k_tile + st * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + (uint32_t)(g * 128), umma_desc_k_sw128(qa + kb * HALF_BYTES + k * 32), umma_desc_k_sw128(ka + kb * HALF_BYTES + k * 32), idesc_s,
                         (kb | k) ? 1u : 0u);
        umma_commit(&sh->s_full[g]);
        const bool last_user = (g == GROUPS - 1) || j >= n_g[GROUPS - 1];
        if (last_user) umma_commit(&sh->k_empty[st]);
        return true;
      };
      // O_g (+)= P_g V_j with P_g read from tensor memory.  V_j is released once the last group that needs it has
      // issued its product.
      auto issue_pv = [&](int g, int j) {
        if (j >= n_g[g]) return true;
        const int st = j & 1;
        if (!mbar_wait(&sh->p_ready[g], (uint32_t)(j & 1), abort_flag)) return false;
        if (v_seen < j) {
          if (!mbar_wait(&sh->v_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
          v_seen = j;
        }
        tc_fence_after();
        const uint32_t va = smem_u32(v_tile + st * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ts(tmem + 256u + (uint32_t)(g * 128), tmem + (uint32_t)(g * 128) + (uint32_t)(ks * 8), umma_desc_mn_sw128(va + ks * 2048, lbo, sbo), idesc_o,
                       (j | ks) ? 1u : 0u);
        umma_commit(&sh->o_full[g]);
        const bool last_user = (g == GROUPS - 1) || j >= n_g[GROUPS - 1];
        if (last_user) umma_commit(&sh->v_empty[st]);
        return true;
      };
      ok = ok && issue_s(0, 0) && issue_s(1, 0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // while one group's softmax runs, the tensor core has the other group's product and next scores to do
        ok = issue_pv(0, j) && issue_s(0, j + 1) && issue_pv(1, j) && issue_s(1, j + 1);
      }
    }
  } else {
    // softmax / output warps: group g = one query tile, one row per thread (TMEM lane 32 * (warp % 4) + lane)
    const int g = (warp - 2) >> 2, wq = warp & 3;
    const int r = wq * 32 + lane;
    const int my_n = n_g[g];
    const int pos0 = pos_base + g * 128;  // position of the group's first row
    const int my_pos = pos0 + r;          // rows past the sequence compute garbage that is never stored
    const uint32_t s_row = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(g * 128);
    const uint32_t o_row = s_row + 256u;
    float m = -INFINITY, l = 0.f;  // m: the maximum the exponentials refer to (may lag the true maximum by up to 2^8)
    bool ok = true;
    // One key tile of this group.  MASK (a tile that the causal edge or the end of the keys crosses) is a compile-time
    // property: the plain tiles, nearly all of them, carry no compare or select per element.
    auto tile = [&](int j, auto mask_tag) -> bool {
      constexpr bool MASK = decltype(mask_tag)::value;
      if (!mbar_wait(&sh->s_full[g], (uint32_t)(j & 1), abort_flag)) return false;
      tc_fence_after();
      const int limit = min(my_pos, kv_len - 1) - j * BKV;  // columns 0 .. limit are visible to this row
      // the whole row of S goes to registers in one round trip (four loads in flight, one wait): both the maximum
      // and the exponentials work from there, and S in tensor memory may be overwritten by P right away
      uint32_t v[BKV];
      tmem_ld32(s_row, v);
      tmem_ld32(s_row + 32, v + 32);
      tmem_ld32(s_row + 64, v + 64);
      tmem_ld32(s_row + 96, v + 96);
      tmem_ld_wait();
      float mx_raw;
      if constexpr (MASK) {
        mx_raw = -INFINITY;
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (i <= limit) mx_raw = fmaxf(mx_raw, __uint_as_float(v[i]));
      } else {
        // three-input maximum, four chains instead of one long one
        float m0 = max3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
        float m1 = max3(__uint_as_float(v[3]), __uint_as_float(v[4]), __uint_as_float(v[5]));
        float m2 = max3(__uint_as_float(v[6]), __uint_as_float(v[7]), __uint_as_float(v[8]));
        float m3 = max3(__uint_as_float(v[9]), __uint_as_float(v[10]), __uint_as_float(v[11]));
#pragma unroll
        for (int i = 12; i + 7 < BKV; i += 8) {
          m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
          m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
          m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
          m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
        }
        // 12 + 8 * 14 = 124: four columns left
        m0 = max3(m0, __uint_as_float(v[124]), __uint_as_float(v[125]));
        m1 = max3(m1, __uint_as_float(v[126]), __uint_as_float(v[127]));
        mx_raw = fmaxf(max3(m0, m1, m2), m3);
      }
      const float mx = mx_raw * p.scale_log2;
      // the previous product of this group must be complete before O is rescaled
      if (j >= 1) {
        if (!mbar_wait(&sh->o_full[g], (uint32_t)((j - 1) & 1), abort_flag)) return false;
        tc_fence_after();
      }
      // move to a new maximum only when it grew by more than the threshold (or there was none yet)
      float alpha = 1.f;
      if (mx > m + RESCALE_LOG2 || (m == -INFINITY && mx > -INFINITY)) {
        alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - mx);
        m = mx;
      }
      if (j >= 1 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) {
        const float2 a2 = make_float2(alpha, alpha);
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t w[32];
          tmem_ld32(o_row + c, w);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 t2 = __fmul2_rn(make_float2(__uint_as_float(w[i]), __uint_as_float(w[i + 1])), a2);
            w[i] = __float_as_uint(t2.x);
            w[i + 1] = __float_as_uint(t2.y);
          }
          tmem_st16(o_row + c, w);
          tmem_st16(o_row + c + 16, w + 16);
        }
        l *= alpha;
      }
      const float neg = (m == -INFINITY) ? 0.f : -m;
      // P = exp2(S * scale - m) as bf16, two per 32-bit column, over the first 64 columns of S; row sum
      float2 sum2 = make_float2(0.f, 0.f), sum3 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), ng2 = make_float2(neg, neg);
#pragma unroll
      for (int c = 0; c < BKV; c += 32) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float2 t2 = __ffma2_rn(make_float2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1])), sc2, ng2);
          const float2 t3 = __ffma2_rn(make_float2(__uint_as_float(v[c + i + 2]), __uint_as_float(v[c + i + 3])), sc2, ng2);
          float2 e = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
          float2 f = make_float2(ex2_approx(t3.x), ex2_approx(t3.y));
          if constexpr (MASK) {
            if (c + i > limit) e.x = 0.f;
            if (c + i + 1 > limit) e.y = 0.f;
            if (c + i + 2 > limit) f.x = 0.f;
            if (c + i + 3 > limit) f.y = 0.f;
          }
          sum2 = __fadd2_rn(sum2, e);
          sum3 = __fadd2_rn(sum3, f);
          const bf162 pe = __floats2bfloat162_rn(e.x, e.y), pf = __floats2bfloat162_rn(f.x, f.y);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pe);
          packed[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&pf);
        }
        tmem_st16(s_row + (c >> 1), packed);
      }
      sum2 = __fadd2_rn(sum2, sum3);
      tmem_st_wait();
      l += sum2.x + sum2.y;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_ready[g]);
      return true;
    };
    for (int j = 0; j < my_n && ok; ++j) {
      const bool need_mask = j * BKV + BKV - 1 > min(pos0, kv_len - 1);
      ok = need_mask ? tile(j, std::true_type{}) : tile(j, std::false_type{});
    }
    const int rows_g = min(128, rows_here - g * 128);
    if (ok && my_n > 0) {
      ok = mbar_wait(&sh->o_full[g], (uint32_t)((my_n - 1) & 1), abort_flag);
      tc_fence_after();
    }
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    bf16* dst = p.out + ((long long)(q0 + row_base + g * 128 + r) * p.hq + hq) * D;
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      uint32_t w[32];
      if (my_n > 0) {  // uniform per group
        tmem_ld32(o_row + c, w);
        tmem_ld_wait();
      }
      if (r < rows_g) {
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = my_n > 0 ? __uint_as_float(w[c8 + i]) * inv : 0.f;
          *reinterpret_cast<bf16x8*>(dst + c + c8) = pack8(f);
        }
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


// ---------------------------------------------------------------------------------------------------------------------
// Head dim 256 (the gated full-attention layers of the hybrid models).  O of one 128-row query tile already takes 256 of
// the 512 TMEM columns, so a CTA owns ONE query tile and keeps the tensor core busy the other way round: the scores are
// double-buffered (tiles of 64 keys, S_j at columns 256 + 64 (j & 1)), and the MMA thread issues  P V of tile j, then S of
// tile j + 2  while the softmax warps work on tile j + 1.  Shared memory: Q 64 KB, K and V two stages of 32 KB each.
// The producer warp is split: lanes 0-15 feed K, lanes 16-31 feed V, each half with its own waits, because K runs two
// tiles ahead of V.
constexpr int D2 = 256, BKV2 = 64, BQ1 = 128;
constexpr int Q2_BYTES = BQ1 * D2 * 2;     // 64 KB: [4 blocks of 64 columns][128 rows][128 B]
constexpr int KV2_BYTES = BKV2 * D2 * 2;   // 32 KB: [4 blocks of 64 columns][64 rows][128 B]
constexpr int KV2_BLOCK = BKV2 * 128;      // 8 KB
constexpr int THREADS2 = 64 + 128;

// One tile of 64 keys for one query row per thread (the head-dim-256 and MLA kernels): S of the tile -> registers ->
// maximum -> lazy rescale of O (`o_cols` columns at `o_row`) -> P as bf16 over the first 32 columns of S -> `p_ready`.
// `o_full` / `o_parity` name the completion of the previous product into the same O (ignored for j == 0).
template <bool MASK>
__device__ __forceinline__ bool softmax_tile64(uint64_t* s_full, uint32_t s_parity, uint32_t s_row, uint32_t o_row, int o_cols, uint64_t* o_full, uint32_t o_parity, int j, int limit, int lo,
                                               float scale_log2, float& m, float& l, uint64_t* p_ready, int lane, volatile int* abort_flag) {
  if (!mbar_wait(s_full, s_parity, abort_flag)) return false;
  tc_fence_after();
  uint32_t v[BKV2];
  tmem_ld32(s_row, v);
  tmem_ld32(s_row + 32, v + 32);
  tmem_ld_wait();
  float mx_raw;
  if constexpr (MASK) {
    mx_raw = -INFINITY;
#pragma unroll
    for (int i = 0; i < BKV2; ++i)
      if (i <= limit && i > lo) mx_raw = fmaxf(mx_raw, __uint_as_float(v[i]));
  } else {
    float m0 = max3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
    float m1 = max3(__uint_as_float(v[3]), __uint_as_float(v[4]), __uint_as_float(v[5]));
    float m2 = max3(__uint_as_float(v[6]), __uint_as_float(v[7]), __uint_as_float(v[8]));
    float m3 = max3(__uint_as_float(v[9]), __uint_as_float(v[10]), __uint_as_float(v[11]));
#pragma unroll
    for (int i = 12; i + 7 < BKV2; i += 8) {
      m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
      m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
      m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
    }
    // 12 + 8 * 6 = 60: four columns left
    m0 = max3(m0, __uint_as_float(v[60]), __uint_as_float(v[61]));
    m1 = max3(m1, __uint_as_float(v[62]), __uint_as_float(v[63]));
    mx_raw = fmaxf(max3(m0, m1, m2), m3);
  }
  const float mx = mx_raw * scale_log2;
  // the previous product must be complete before O is rescaled
  if (j >= 1) {
    if (!mbar_wait(o_full, o_parity, abort_flag)) return false;
    tc_fence_after();
  }
  float alpha = 1.f;
  if (mx > m + RESCALE_LOG2 || (m == -INFINITY && mx > -INFINITY)) {
    alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - mx);
    m = mx;
  }
  if (j >= 1 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) {
    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll 1
    for (int c = 0; c < o_cols; c += 32) {
      uint32_t w[32];
      tmem_ld32(o_row + c, w);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 t2 = __fmul2_rn(make_float2(__uint_as_float(w[i]), __uint_as_float(w[i + 1])), a2);
        w[i] = __float_as_uint(t2.x);
        w[i + 1] = __float_as_uint(t2.y);
      }
      tmem_st16(o_row + c, w);
      tmem_st16(o_row + c + 16, w + 16);
    }
    l *= alpha;
  }
  const float neg = (m == -INFINITY) ? 0.f : -m;
  float2 sum2 = make_float2(0.f, 0.f), sum3 = make_float2(0.f, 0.f);
  const float2 sc2 = make_float2(scale_log2, scale_log2), ng2 = make_float2(neg, neg);
#pragma unroll
  for (int c = 0; c < BKV2; c += 32) {
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float2 t2 = __ffma2_rn(make_float2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1])), sc2, ng2);
      const float2 t3 = __ffma2_rn(make_float2(__uint_as_float(v[c + i + 2]), __uint_as_float(v[c + i + 3])), sc2, ng2);
      float2 e = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
      float2 f = make_float2(ex2_approx(t3.x), ex2_approx(t3.y));
      if constexpr (MASK) {
        if (c + i > limit || c + i <= lo) e.x = 0.f;
        if (c + i + 1 > limit || c + i + 1 <= lo) e.y = 0.f;
        if (c + i + 2 > limit || c + i + 2 <= lo) f.x = 0.f;
        if (c + i + 3 > limit || c + i + 3 <= lo) f.y = 0.f;
      }
      sum2 = __fadd2_rn(sum2, e);
      sum3 = __fadd2_rn(sum3, f);
      const bf162 pe = __floats2bfloat162_rn(e.x, e.y), pf = __floats2bfloat162_rn(f.x, f.y);
      packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pe);
      packed[(i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&pf);
    }
    tmem_st16(s_row + (c >> 1), packed);
  }
  sum2 = __fadd2_rn(sum2, sum3);
  tmem_st_wait();
  l += sum2.x + sum2.y;
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(p_ready);
  return true;
}


struct TcSmem2 {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_full;
  uint32_t tmem_slot;
  int abort_flag;
};

__global__ void __launch_bounds__(THREADS2, 1) prefill_attn_tc256_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* q_tile = tiles;
  uint8_t* k_tile = tiles + Q2_BYTES;
  uint8_t* v_tile = k_tile + 2 * KV2_BYTES;
  TcSmem2* sh = reinterpret_cast<TcSmem2*>(v_tile + 2 * KV2_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = (int)(blockIdx.x % (unsigned)p.hq);
  const int h = hq / (p.hq / p.hkv);
  int b = 0, tile_in_seq = 0;  // late tiles (most keys) first, every head's before any early tile
  {
    int rem = (int)(gridDim.x / (unsigned)p.hq) - 1 - (int)(blockIdx.x / (unsigned)p.hq);
    for (; b < p.num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + BQ1 - 1) / BQ1;
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
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(&sh->k_full[s2], 1);
      mbar_init(&sh->k_empty[s2], 1);
      mbar_init(&sh->v_full[s2], 1);
      mbar_init(&sh->v_empty[s2], 1);
      mbar_init(&sh->s_full[s2], 1);
      mbar_init(&sh->p_ready[s2], 4);
    }
    mbar_init(&sh->o_full, 1);
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
  const uint32_t tmem = sh->tmem_slot;  // columns: O at 0 .. 255, S / P of tile j at 256 + 64 (j & 1)
  volatile int* abort_flag = &sh->abort_flag;
  PG_PDL_ENTRY();

  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int row_base = tile_in_seq * BQ1;
  const int rows_here = min(BQ1, q_len - row_base);
  const int pos0 = kv_len - q_len + row_base;  // position of the tile's first row
  // key tiles j0 .. last the rows of this tile can see (a sliding window drops the tiles in front of the first row's
  // window); the loops below count tiles from j0
  const int j0 = (p.window > 0 && rows_here > 0) ? max(0, pos0 - p.window + 1) / BKV2 : 0;
  const int n_tiles = (rows_here > 0 && kv_len > 0) ? min(pos0 + rows_here - 1, kv_len - 1) / BKV2 + 1 - j0 : 0;
  const int* table_row = p.table + (long long)b * p.table_stride;

  if (warp == 0) {
    if (n_tiles > 0) {
      const uint64_t pol = l2_policy_evict_normal();
      if (lane == 0) {
        mbar_expect_tx(&sh->q_full, Q2_BYTES);
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) tma_load_3d(q_tile + cb * (BQ1 * 128), &tm_q, &sh->q_full, cb * 64, hq, q0 + row_base, pol);
      }
      // lanes 0-15: K boxes, lanes 16-31: V boxes; slot = (page of the tile, 64-column block), 4 * ppt slots per tile
      const int kvsel = lane >> 4, sub = lane & 15;
      const uint32_t half_mask = kvsel ? 0xFFFF0000u : 0x0000FFFFu;
      const int ppt = BKV2 / p.page_size;  // 1 .. 8
      const int slots = 4 * ppt;           // 4 .. 32: up to two per lane
      uint64_t* full = kvsel ? sh->v_full : sh->k_full;
      uint64_t* empty = kvsel ? sh->v_empty : sh->k_empty;
      uint8_t* tile0 = kvsel ? v_tile : k_tile;
      auto page_of = [&](int j, int slot) -> int {
        const int pg = slot >> 2;
        const int pages_live = min(ppt, (kv_len - j * BKV2 + p.page_size - 1) / p.page_size);
        int page = (slot < slots && pg < pages_live) ? __ldg(table_row + j * ppt + pg) : 0;  // past the end: the padding page, keys masked
        if (page < 0 || page >= p.num_pages) {
          atomicCAS(p.status, PG_ST_OK, PG_ST_BOUNDS | (42u << 8));
          page = 0;
        }
        return page;
      };
      int nxt0 = page_of(j0, sub), nxt1 = page_of(j0, sub + 16);
      for (int j = 0; j < n_tiles; ++j) {
        const int pg0 = nxt0, pg1 = nxt1;
        if (j + 1 < n_tiles) {
          nxt0 = page_of(j0 + j + 1, sub);
          nxt1 = page_of(j0 + j + 1, sub + 16);
        }
        const int st = j & 1;
        if (j >= 2) {
          bool ok = mbar_wait(&empty[st], (uint32_t)(((j >> 1) - 1) & 1), abort_flag);
          ok = __all_sync(half_mask, ok);
          if (!ok) break;
        }
        if (sub == 0) mbar_expect_tx(&full[st], KV2_BYTES);
        __syncwarp(half_mask);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int slot = sub + 16 * it;
          if (slot < slots) {
            const int pg = slot >> 2, cb = slot & 3;
            const int z = ((it ? pg1 : pg0) * 2 + kvsel) * p.page_size;
            tma_load_3d(tile0 + st * KV2_BYTES + cb * KV2_BLOCK + pg * p.page_size * 128, &tm_kv, &full[st], cb * 64, h, z, pol);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, BKV2, 0);
      constexpr uint32_t idesc_o = idesc_bf16(128, D2, 1);
      const uint32_t lbo = p.mn_lbo_first ? (uint32_t)KV2_BLOCK : 1024u, sbo = p.mn_lbo_first ? 1024u : (uint32_t)KV2_BLOCK;
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      // S of tile j into buffer j & 1.  It overwrites S and P of tile j - 2: the product that read that P was issued
      // before, and the tensor core runs this thread's instructions in order.
      auto issue_s = [&](int j) {
        if (j >= n_tiles) return true;
        const int st = j & 1;
        if (!mbar_wait(&sh->k_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(q_tile), ka = smem_u32(k_tile + st * KV2_BYTES);
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + 256u + (uint32_t)(st * BKV2), umma_desc_k_sw128(qa + cb * (BQ1 * 128) + k * 32), umma_desc_k_sw128(ka + cb * KV2_BLOCK + k * 32), idesc_s,
                         (cb | k) ? 1u : 0u);
        umma_commit(&sh->s_full[st]);
        umma_commit(&sh->k_empty[st]);
        return true;
      };
      ok = ok && issue_s(0) && issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        ok = mbar_wait(&sh->p_ready[st], (uint32_t)((j >> 1) & 1), abort_flag) && mbar_wait(&sh->v_full[st], (uint32_t)((j >> 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(v_tile + st * KV2_BYTES);
#pragma unroll
        for (int ks = 0; ks < BKV2 / 16; ++ks)
          umma_bf16_ts(tmem, tmem + 256u + (uint32_t)(st * BKV2) + (uint32_t)(ks * 8), umma_desc_mn_sw128(va + ks * 2048, lbo, sbo), idesc_o, (j | ks) ? 1u : 0u);
        umma_commit(&sh->o_full);
        umma_commit(&sh->v_empty[st]);
        ok = issue_s(j + 2);
      }
    }
  } else {
    // softmax / output warps: one query row per thread (TMEM lane 32 * (warp % 4) + lane)
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const int my_pos = pos0 + r;  // rows past the sequence compute garbage that is never stored
    const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_row = lane_base;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int key0 = (j0 + j) * BKV2;
      // a tile needs the mask when the causal edge or the end of the keys crosses it, or (sliding window) when its first
      // key lies in front of the window of the tile's last row
      const bool need_mask = key0 + BKV2 - 1 > min(pos0, kv_len - 1) || (p.window > 0 && key0 <= pos0 + BQ1 - 1 - p.window);
      const int st = j & 1;
      const uint32_t s_row = lane_base + 256u + (uint32_t)(st * BKV2);
      const int limit = min(my_pos, kv_len - 1) - key0;                          // columns lo + 1 .. limit are visible to this row
      const int lo = p.window > 0 ? my_pos - p.window - key0 : -(1 << 30);
      const uint32_t sp = (uint32_t)((j >> 1) & 1), op = (uint32_t)((j - 1) & 1);
      ok = need_mask ? softmax_tile64<true>(&sh->s_full[st], sp, s_row, o_row, D2, &sh->o_full, op, j, limit, lo, p.scale_log2, m, l, &sh->p_ready[st], lane, abort_flag)
                     : softmax_tile64<false>(&sh->s_full[st], sp, s_row, o_row, D2, &sh->o_full, op, j, limit, lo, p.scale_log2, m, l, &sh->p_ready[st], lane, abort_flag);
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(&sh->o_full, (uint32_t)((n_tiles - 1) & 1), abort_flag);
      tc_fence_after();
    }
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    bf16* dst = p.out + ((long long)(q0 + row_base + r) * p.hq + hq) * D2;
#pragma unroll 1
    for (int c = 0; c < D2; c += 32) {
      uint32_t w[32];
      if (n_tiles > 0) {
        tmem_ld32(o_row + c, w);
        tmem_ld_wait();
      }
      if (r < rows_here) {
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = n_tiles > 0 ? __uint_as_float(w[c8 + i]) * inv : 0.f;
          *reinterpret_cast<bf16x8*>(dst + c + c8) = pack8(f);
        }
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
  if (threadIdx.x == 0 && sh->abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (42u << 8));
}


// ---------------------------------------------------------------------------------------------------------------------
// Multi-head latent attention, prefill, in the expanded (not absorbed) form: per head, queries and keys of 128 + 64
// (rotary part, one key row shared by all heads) and values of 128, keys and values dense rows [sum of kv lengths, heads,
// 128] that the caller expanded from the gathered latent rows with the up-projection GEMMs.  The absorbed form the decode
// kernel uses would contract over 576 and accumulate 512 columns per row; expanded, a prefill chunk costs a quarter of
// the FLOPs and O fits tensor memory.  Structure as for head dim 128 (two query tiles of 128 rows per CTA whose softmax
// groups alternate on the tensor core, P in tensor memory), with key tiles of 64 so that Q (2 x 48 KB) and two stages of
// K (24 KB) and V (16 KB) fit shared memory.  The rotary block of Q and K comes through tensor maps of its own.
//
// Reference parity: pegainfer-kernels/csrc/k3/k3_flash_mla_prefill.cu (gather / expand, then a dense SM100 FMHA).
constexpr int MQ_BYTES = 128 * 192 * 2;  // 48 KB: [3 blocks of 64 columns][128 rows][128 B]
constexpr int MK_BYTES = BKV2 * 192 * 2; // 24 KB: [3 blocks][64 rows][128 B]
constexpr int MV_BYTES = BKV2 * 128 * 2; // 16 KB: [2 blocks][64 rows][128 B]

struct MlaTcParams {
  bf16* out;             // [T, heads * 128]
  const int* q_indptr;   // [num_seqs + 1]
  const int* kv_indptr;  // [num_seqs + 1] rows of the dense K / V
  const int* kv_lens;    // [num_seqs]
  int num_seqs, heads;
  float scale_log2;
  int mn_lbo_first;
  uint32_t* status;
};

__global__ void __launch_bounds__(THREADS, 1) mla_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qpe,
                                                                    const __grid_constant__ CUtensorMap tm_kn, const __grid_constant__ CUtensorMap tm_kpe,
                                                                    const __grid_constant__ CUtensorMap tm_v, const MlaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* tiles = smem_raw + (((base + 1023u) & ~1023u) - base);
  uint8_t* q_tile = tiles;                    // GROUPS x 48 KB
  uint8_t* k_tile = tiles + GROUPS * MQ_BYTES;  // 2 x 24 KB
  uint8_t* v_tile = k_tile + 2 * MK_BYTES;    // 2 x 16 KB
  TcSmem* sh = reinterpret_cast<TcSmem*>(v_tile + 2 * MV_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = (int)(blockIdx.x % (unsigned)p.heads);
  int b = 0, tile_in_seq = 0;  // late tiles (most keys) first, every head's before any early tile
  {
    int rem = (int)(gridDim.x / (unsigned)p.heads) - 1 - (int)(blockIdx.x / (unsigned)p.heads);
    for (; b < p.num_seqs; ++b) {
      const int n = p.q_indptr[b + 1] - p.q_indptr[b];
      const int nt = (n + BQ2 - 1) / BQ2;
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
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(&sh->k_full[s2], 1);
      mbar_init(&sh->k_empty[s2], 1);
      mbar_init(&sh->v_full[s2], 1);
      mbar_init(&sh->v_empty[s2], 1);
    }
    for (int g = 0; g < GROUPS; ++g) {
      mbar_init(&sh->s_full[g], 1);
      mbar_init(&sh->p_ready[g], 4);
      mbar_init(&sh->o_full[g], 1);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_qn);
    tma_prefetch_desc(&tm_qpe);
    tma_prefetch_desc(&tm_kn);
    tma_prefetch_desc(&tm_kpe);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;  // columns: S / P of group g at 128 g (64 used), O of group g at 256 + 128 g
  volatile int* abort_flag = &sh->abort_flag;
  PG_PDL_ENTRY();

  const int q0 = p.q_indptr[b], q_len = p.q_indptr[b + 1] - q0;
  const int kv_len = p.kv_lens[b], kv0 = p.kv_indptr[b];
  const int row_base = tile_in_seq * BQ2;
  const int rows_here = min(BQ2, q_len - row_base);
  const int pos_base = kv_len - q_len + row_base;
  int n_g[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int rows_of_g = min(128, rows_here - g * 128);
    n_g[g] = (rows_of_g > 0 && kv_len > 0) ? min(pos_base + g * 128 + rows_of_g - 1, kv_len - 1) / BKV2 + 1 : 0;
  }
  const int n_tiles = max(n_g[0], n_g[1]);

  if (warp == 0) {
    if (n_tiles > 0) {
      const uint64_t pol = l2_policy_evict_normal();
      if (lane == 0) {
        mbar_expect_tx(&sh->q_full, GROUPS * MQ_BYTES);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          const int row = q0 + row_base + g * 128;
          tma_load_3d(q_tile + g * MQ_BYTES, &tm_qn, &sh->q_full, 0, row, h, pol);            // nope columns 0 .. 63   ([heads, T, 128])
          tma_load_3d(q_tile + g * MQ_BYTES + 16384, &tm_qn, &sh->q_full, 64, row, h, pol);   // nope columns 64 .. 127
          tma_load_3d(q_tile + g * MQ_BYTES + 32768, &tm_qpe, &sh->q_full, 0, h, row, pol);   // rotary part            ([T, heads, 64])
        }
      }
      // five boxes per tile, one lane each: K nope (2), K rotary, V (2)
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const int row = kv0 + j * BKV2;  // rows past the sequence belong to the next one (or are filled with zeros): masked
        if (j >= 2) {
          const uint32_t par = (uint32_t)(((j >> 1) - 1) & 1);
          ok = mbar_wait(&sh->k_empty[st], par, abort_flag) && mbar_wait(&sh->v_empty[st], par, abort_flag);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
        }
        if (lane == 0) {
          mbar_expect_tx(&sh->k_full[st], MK_BYTES);
          mbar_expect_tx(&sh->v_full[st], MV_BYTES);
        }
        __syncwarp();
        if (lane < 2) tma_load_3d(k_tile + st * MK_BYTES + lane * 8192, &tm_kn, &sh->k_full[st], lane * 64, h, row, pol);
        else if (lane == 2) tma_load_2d(k_tile + st * MK_BYTES + 16384, &tm_kpe, &sh->k_full[st], 0, row, pol);
        else if (lane < 5) tma_load_3d(v_tile + st * MV_BYTES + (lane - 3) * 8192, &tm_v, &sh->v_full[st], (lane - 3) * 64, h, row, pol);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, BKV2, 0);
      constexpr uint32_t idesc_o = idesc_bf16(128, 128, 1);
      const uint32_t lbo = p.mn_lbo_first ? 8192u : 1024u, sbo = p.mn_lbo_first ? 1024u : 8192u;
      bool ok = mbar_wait(&sh->q_full, 0, abort_flag);
      int k_seen = -1, v_seen = -1;
      auto issue_s = [&](int g, int j) {
        if (j >= n_g[g]) return true;
        const int st = j & 1;
        if (k_seen < j) {
          if (!mbar_wait(&sh->k_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
          k_seen = j;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(q_tile + g * MQ_BYTES), ka = smem_u32(k_tile + st * MK_BYTES);
#pragma unroll
        for (int cb = 0; cb < 3; ++cb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem + (uint32_t)(g * 128), umma_desc_k_sw128(qa + cb * 16384 + k * 32), umma_desc_k_sw128(ka + cb * 8192 + k * 32), idesc_s, (cb | k) ? 1u : 0u);
        umma_commit(&sh->s_full[g]);
        const bool last_user = (g == GROUPS - 1) || j >= n_g[GROUPS - 1];
        if (last_user) umma_commit(&sh->k_empty[st]);
        return true;
      };
      auto issue_pv = [&](int g, int j) {
        if (j >= n_g[g]) return true;
        const int st = j & 1;
        if (!mbar_wait(&sh->p_ready[g], (uint32_t)(j & 1), abort_flag)) return false;
        if (v_seen < j) {
          if (!mbar_wait(&sh->v_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
          v_seen = j;
        }
        tc_fence_after();
        const uint32_t va = smem_u32(v_tile + st * MV_BYTES);
#pragma unroll
        for (int ks = 0; ks < BKV2 / 16; ++ks)
          umma_bf16_ts(tmem + 256u + (uint32_t)(g * 128), tmem + (uint32_t)(g * 128) + (uint32_t)(ks * 8), umma_desc_mn_sw128(va + ks * 2048, lbo, sbo), idesc_o, (j | ks) ? 1u : 0u);
        umma_commit(&sh->o_full[g]);
        const bool last_user = (g == GROUPS - 1) || j >= n_g[GROUPS - 1];
        if (last_user) umma_commit(&sh->v_empty[st]);
        return true;
      };
      ok = ok && issue_s(0, 0) && issue_s(1, 0);
      for (int j = 0; j < n_tiles && ok; ++j) ok = issue_pv(0, j) && issue_s(0, j + 1) && issue_pv(1, j) && issue_s(1, j + 1);
    }
  } else {
    const int g = (warp - 2) >> 2, wq = warp & 3;
    const int r = wq * 32 + lane;
    const int my_n = n_g[g];
    const int pos0 = pos_base + g * 128;
    const int my_pos = pos0 + r;
    const uint32_t s_row = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(g * 128);
    const uint32_t o_row = s_row + 256u;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_n && ok; ++j) {
      const bool need_mask = j * BKV2 + BKV2 - 1 > min(pos0, kv_len - 1);
      const int limit = min(my_pos, kv_len - 1) - j * BKV2;
      const uint32_t sp = (uint32_t)(j & 1), op = (uint32_t)((j - 1) & 1);
      ok = need_mask ? softmax_tile64<true>(&sh->s_full[g], sp, s_row, o_row, 128, &sh->o_full[g], op, j, limit, -(1 << 30), p.scale_log2, m, l, &sh->p_ready[g], lane, abort_flag)
                     : softmax_tile64<false>(&sh->s_full[g], sp, s_row, o_row, 128, &sh->o_full[g], op, j, limit, -(1 << 30), p.scale_log2, m, l, &sh->p_ready[g], lane, abort_flag);
    }
    const int rows_g = min(128, rows_here - g * 128);
    if (ok && my_n > 0) {
      ok = mbar_wait(&sh->o_full[g], (uint32_t)((my_n - 1) & 1), abort_flag);
      tc_fence_after();
    }
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    bf16* dst = p.out + ((long long)(q0 + row_base + g * 128 + r) * p.heads + h) * 128;
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t w[32];
      if (my_n > 0) {  // uniform per group
        tmem_ld32(o_row + c, w);
        tmem_ld_wait();
      }
      if (r < rows_g) {
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = my_n > 0 ? __uint_as_float(w[c8 + i]) * inv : 0.f;
          *reinterpret_cast<bf16x8*>(dst + c + c8) = pack8(f);
        }
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
  if (threadIdx.x == 0 && sh->abort_flag) atomicCAS(p.status, PG_ST_OK, PG_ST_TIMEOUT | (43u << 8));
}

// Latent rows of every key of the step's sequences, through the page table, as dense rows [sum of kv lengths, width].
__global__ void __launch_bounds__(128) mla_gather_latent_kernel(const bf16* __restrict__ latent, int page_size, long long num_pages, int width, const int* __restrict__ table,
                                                                int table_stride, const int* __restrict__ kv_indptr, int num_seqs, bf16* __restrict__ out, uint32_t* status) {
  const int row = blockIdx.x;
  int b = 0;
  while (b + 1 < num_seqs && kv_indptr[b + 1] <= row) ++b;
  const int pos = row - kv_indptr[b];
  int page = table[(long long)b * table_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicCAS(status, PG_ST_OK, PG_ST_BOUNDS | (44u << 8));
    page = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(latent + ((long long)page * page_size + pos % page_size) * width);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)row * width);
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
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

// [rows, heads, dim] bf16, contiguous; box = 64 columns x 1 head x box_rows rows, 128-byte swizzle
int make_tmap_rows_heads(CUtensorMap* out, const void* ptr, long long rows, int heads, int box_rows, int dim = D) {
  EncodeTiledFn enc = get_encode_attn();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0, "TMA base address must be 16-byte aligned");
  cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)dim * 2, (cuuint64_t)heads * dim * 2};
  cuuint32_t box[3] = {64u, 1u, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}


// generic tiled tensor map over bf16 with the 128-byte swizzle (inner box = 64 elements)
int make_tmap_bf16(CUtensorMap* out, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box) {
  EncodeTiledFn enc = get_encode_attn();
  PG_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  PG_REQUIRE(((uintptr_t)ptr & 15) == 0, "TMA base address must be 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i) PG_REQUIRE(strides_bytes[i] % 16 == 0, "TMA stride %d of %llu bytes is not a multiple of 16", i, (unsigned long long)strides_bytes[i]);
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PG_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return PG_OK;
}

int g_mn_variant = -1;

}  // namespace

// Test hook: which of the two stride fields of the MN-major descriptor carries the 64-column block stride.
extern "C" void pg_prefill_attention_tc_variant(int v) { g_mn_variant = v; }

// q [T, hq, d] bf16 (contiguous), kv_layer [pages, 2, page_size, hkv, d], out [T, hq * d], d = 128 or 256.  `q_tiles` = sum
// over the sequences of ceil(query rows / 256) for d = 128 and of ceil(query rows / 128) for d = 256.
extern "C" int pg_prefill_attention_tc(const void* q, const void* kv_layer, void* out, const void* q_indptr, const void* kv_lens, const void* table, int table_stride,
                                       int num_seqs, int tokens, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int q_tiles, int window,
                                       void* status, cudaStream_t stream) {
  PG_REQUIRE(window == 0 || dim == D2, "tcgen05 prefill attention: a sliding window is built for head dim 256 only");
  PG_REQUIRE(dim == D || dim == D2, "tcgen05 prefill attention is built for head dims 128 and 256 (got %d)", dim);
  const int key_tile = dim == D ? BKV : BKV2;
  PG_REQUIRE(page_size >= 8 && page_size <= key_tile && key_tile % page_size == 0, "page size %d does not tile %d keys", page_size, key_tile);
  PG_REQUIRE(num_pages * 2 * page_size < (1ll << 31), "KV cache of %lld pages is too large for 32-bit TMA row coordinates", num_pages);
  PG_REQUIRE(hq % hkv == 0, "query heads %d are not a multiple of the KV heads %d", hq, hkv);
  if (q_tiles == 0 || tokens == 0) return PG_OK;
  CUtensorMap tm_q, tm_kv;
  int rc = make_tmap_rows_heads(&tm_q, q, tokens, hq, 128, dim);
  if (rc != PG_OK) return rc;
  rc = make_tmap_rows_heads(&tm_kv, kv_layer, num_pages * 2 * page_size, hkv, page_size, dim);
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
  p.window = window;
  p.mn_lbo_first = g_mn_variant < 0 ? 1 : g_mn_variant;
  p.status = (uint32_t*)status;
  if (dim == D2) {
    const size_t smem2 = 1024 + (size_t)Q2_BYTES + 4 * (size_t)KV2_BYTES + sizeof(TcSmem2) + 64;
    static bool attr2_done = false;
    if (!attr2_done) {
      PG_CUDA(cudaFuncSetAttribute(prefill_attn_tc256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
      attr2_done = true;
    }
    PG_CUDA(launch_pdl(prefill_attn_tc256_kernel, dim3((unsigned)q_tiles * (unsigned)hq), dim3(THREADS2), smem2, stream, tm_q, tm_kv, p));
    PG_LAUNCH_CHECK();
    return PG_OK;
  }
  const size_t smem = 1024 + (GROUPS + 4) * (size_t)TILE_BYTES + sizeof(TcSmem) + 64;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(prefill_attn_tc_kernel, dim3((unsigned)q_tiles * (unsigned)hq), dim3(THREADS), smem, stream, tm_q, tm_kv, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// Dense latent rows of the step's keys: latent_layer [pages, page_size, width] -> out [total_kv, width].
extern "C" int pg_mla_gather_latent(const void* latent_layer, int page_size, long long num_pages, int width, const void* table, int table_stride, const void* kv_indptr,
                                    int num_seqs, int total_kv, void* out, void* status, cudaStream_t stream) {
  PG_REQUIRE(width % 8 == 0, "latent width %d is not a multiple of 8", width);
  if (total_kv == 0) return PG_OK;
  PG_CUDA(launch_pdl(mla_gather_latent_kernel, dim3((unsigned)total_kv), dim3(128), 0, stream, (const bf16*)latent_layer, page_size, num_pages, width, (const int*)table,
                     table_stride, (const int*)kv_indptr, num_seqs, (bf16*)out, (uint32_t*)status));
  PG_LAUNCH_CHECK();
  return PG_OK;
}

// Expanded-form MLA prefill on tcgen05.  q_nope_hm [heads, T, 128] with `q_nope_head_stride` elements between heads (the rows may be
// a prefix of a longer step), q_pe [T, heads, 64], k_nope and v [total_kv, heads, 128],
// k_pe = column `pe_col` of the dense latent rows [total_kv, pe_ld]; out [T, heads * 128].  `q_tiles` = sum over the
// sequences of ceil(query rows / 256).
extern "C" int pg_mla_prefill_tc(const void* q_nope_hm, long long q_nope_head_stride, const void* q_pe, const void* k_nope, const void* k_pe_rows, int pe_ld, int pe_col, const void* v, void* out,
                                 const void* q_indptr, const void* kv_indptr, const void* kv_lens, int num_seqs, int tokens, int total_kv, int heads, int nope, int rope, int vdim,
                                 float scale, int q_tiles, void* status, cudaStream_t stream) {
  PG_REQUIRE(nope == 128 && rope == 64 && vdim == 128, "tcgen05 MLA prefill is built for 128 + 64 query / key and 128 value columns (got %d + %d, %d)", nope, rope, vdim);
  if (q_tiles == 0 || tokens == 0 || total_kv == 0) return PG_OK;
  CUtensorMap tm_qn, tm_qpe, tm_kn, tm_kpe, tm_v;
  {
    cuuint64_t dims[3] = {128, (cuuint64_t)tokens, (cuuint64_t)heads}, st[2] = {128 * 2, (cuuint64_t)q_nope_head_stride * 2};
    cuuint32_t box[3] = {64, 128, 1};
    int rc = make_tmap_bf16(&tm_qn, q_nope_hm, 3, dims, st, box);
    if (rc != PG_OK) return rc;
  }
  {
    cuuint64_t dims[3] = {64, (cuuint64_t)heads, (cuuint64_t)tokens}, st[2] = {64 * 2, (cuuint64_t)heads * 64 * 2};
    cuuint32_t box[3] = {64, 1, 128};
    int rc = make_tmap_bf16(&tm_qpe, q_pe, 3, dims, st, box);
    if (rc != PG_OK) return rc;
  }
  int rc = make_tmap_rows_heads(&tm_kn, k_nope, total_kv, heads, BKV2, 128);
  if (rc != PG_OK) return rc;
  rc = make_tmap_rows_heads(&tm_v, v, total_kv, heads, BKV2, 128);
  if (rc != PG_OK) return rc;
  {
    cuuint64_t dims[2] = {64, (cuuint64_t)total_kv}, st[1] = {(cuuint64_t)pe_ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)BKV2};
    rc = make_tmap_bf16(&tm_kpe, (const bf16*)k_pe_rows + pe_col, 2, dims, st, box);
    if (rc != PG_OK) return rc;
  }
  MlaTcParams p;
  p.out = (bf16*)out;
  p.q_indptr = (const int*)q_indptr;
  p.kv_indptr = (const int*)kv_indptr;
  p.kv_lens = (const int*)kv_lens;
  p.num_seqs = num_seqs;
  p.heads = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mn_lbo_first = g_mn_variant < 0 ? 1 : g_mn_variant;
  p.status = (uint32_t*)status;
  const size_t smem = 1024 + GROUPS * (size_t)MQ_BYTES + 2 * (size_t)MK_BYTES + 2 * (size_t)MV_BYTES + sizeof(TcSmem) + 64;
  static bool attr_done = false;
  if (!attr_done) {
    PG_CUDA(cudaFuncSetAttribute(mla_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  PG_CUDA(launch_pdl(mla_prefill_tc_kernel, dim3((unsigned)q_tiles * (unsigned)heads), dim3(THREADS), smem, stream, tm_qn, tm_qpe, tm_kn, tm_kpe, tm_v, p));
  PG_LAUNCH_CHECK();
  return PG_OK;
}
