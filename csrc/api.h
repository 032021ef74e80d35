// Public C API of libpegainfer_b200.so.  Every entry point returns 0 on success or a
// negative PG_ERR_* code; pg_last_error() then holds a thread-local message.  Pointers
// are device pointers unless named host_*.  `status` arguments are a device uint32 word
// (pg_status_*) that kernels set when a bounded wait expires or an index is out of
// range; kernels never trap.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* pg_last_error(void);
int pg_version(void);

// ---- GEMM (gemm_sm100.cu) ----------------------------------------------------------
int pg_gemm_workspace_bytes(int T, int M, int K, int device, long long* ws_bytes, long long* counter_bytes);
// How a problem would be launched on the current device:
// out[6] = {token tile, k-splits, cluster size, grid, pipeline stages, co-resident clusters of that size}.
int pg_gemm_plan(int T, int M, int K, int force_splits, int* out);
// One-shot hint: the next GEMM launched from the calling thread also pulls `bytes` at `ptr`
// (the weights of the GEMM after it) into L2 with its idle producer lanes.
void pg_gemm_prefetch_next(const void* ptr, long long bytes);
// Profiling hook: device buffer of 16 x uint64 per CTA filled with globaltimer phase stamps by every following GEMM (nullptr = off).
void pg_gemm_set_timing(void* buf);
int pg_gemm_bf16_tn(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                    void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status, int force_splits,
                    cudaStream_t stream);
int pg_gemm_bf16_tn_after_gather(const void* x, const void* w, void* y, int y_is_f32, int T, int M, int K, long long ldx, long long ldw,
                                 long long ldy, void* ws, long long ws_bytes, void* counters, long long counter_bytes, void* status,
                                 const void* wait_flags, int world, unsigned long long wait_ns, cudaStream_t stream);
// Tensor-parallel fused path: GEMM -> reduce-scatter -> +residual -> RMSNorm -> all-gather over NVLink peer memory.
int pg_tp_gemm_rs_norm_ag(const void* a, const void* w, int T, int hidden, int K, long long lda, long long ldw, void* const* part,
                          void* const* xout, void* const* flags, int rank, int world, int site, void* residual, long long ld_res,
                          const void* norm_w, float eps, int offset, int one_shot, long long part_offset, unsigned long long wait_ns, void* ws,
                          long long ws_bytes, void* counters, long long counter_bytes, void* status, cudaStream_t stream);
// Decode-chain GEMM (T <= 64) with the deferred RMSNorm scale of its input rows and a fused epilogue
// (0 plain, 1 SwiGLU over interleaved gate/up rows, 2 residual add + norm-weight product + per-tile sums
// of squares); PG_ERR_UNSUPPORTED when the problem does not plan onto the on-chip split-K path.
int pg_gemm_bf16_tn_fused(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy,
                          const void* in_ssp, int in_parts, int in_ld, int in_width, float in_eps, int epi, void* residual, long long ld_res,
                          const void* norm_w, int norm_offset, void* out_ssp, int out_ld, void* ws, long long ws_bytes, void* counters,
                          long long counter_bytes, void* status, cudaStream_t stream);
// Decode chain (decode_chain.cu): up to four dependent GEMMs of a layer in one persistent kernel for
// steps of at most 64 rows.  One PgChainPhase per GEMM; see decode_chain.cu for the fields.
struct PgChainPhase;
long long pg_decode_chain_ws_bytes(int device);
int pg_decode_chain(const struct PgChainPhase* phases, int nphase, int T, void* residual, long long ld_res, float eps, void* ws, long long ws_bytes,
                    void* counters, void* status, cudaStream_t stream);
// Write a captured cudaGraph_t as Graphviz DOT (graph_export.cu); counts = {nodes, edges, kernel nodes, programmatic edges}.
int pg_graph_export_dot(void* graph, const char* path, const char* title, long long* counts);
int pg_tp_wait(const void* wait_flags, int world, unsigned long long wait_ns, void* status, cudaStream_t stream);
int pg_symm_alloc(long long bytes, void** out);
int pg_symm_free(void* p);
int pg_ipc_export(void* p, void* handle64);
int pg_ipc_import(const void* handle64, void** out);
int pg_ipc_close(void* p);
// Two-SM (cta_group::2) bf16 GEMM for tensor-bound problems (gemm2sm_sm100.cu); pg_gemm_bf16_tn
// routes eligible problems to it (PEGAINFER_GEMM_2SM=0 turns that off).
int pg_gemm2sm_eligible(int T, int M, int K);
int pg_gemm2sm_bf16_tn(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status,
                       cudaStream_t stream);
int pg_gemm2sm_bf16_tn_swiglu(const void* x, const void* w, void* y, int T, int M, int K, long long ldx, long long ldw, long long ldy, void* status,
                       cudaStream_t stream);
int pg_make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols);

// ---- row kernels (elementwise.cu) --------------------------------------------------
int pg_gather_rows(const void* table, const void* ids, void* out, int rows, int width, long long table_rows, void* status, cudaStream_t stream);
int pg_gather_words(const void* src, const void* idx, void* dst, int n, int src_len, void* status, cudaStream_t stream);
int pg_rms_norm(const void* x, void* residual, const void* w, void* y, int rows, int width, float eps, int offset, int round_before,
                long long ldx, long long ldr, long long ldy, cudaStream_t stream);
int pg_gated_rms_norm(const void* x, const void* gate, const void* w_f32, void* y, long long rows, int dim, float eps, cudaStream_t stream);
// act 0: SiLU gate (as above); 1: bf16(norm * w) * bf16(sigmoid(gate))
int pg_gated_rms_norm_act(const void* x, const void* gate, const void* w_f32, void* y, long long rows, int dim, float eps, int act, cudaStream_t stream);
int pg_swiglu(const void* gate_up, void* out, int rows, int inter, long long ldin, long long ldout, int interleaved, cudaStream_t stream);
int pg_sigmoid_gate_mul(void* x, const void* gate, long long n, cudaStream_t stream);
int pg_qk_norm_rope_append(const void* qkv, long long ld, const void* q_w, const void* k_w, const void* cos, const void* sin,
                           const void* positions, const void* slots, void* q_out, void* gate_out, void* kv, int tokens, int hq, int hkv, int dim,
                           int rot, int page_size, long long num_pages, int max_pos, int gated, int offset, float eps, int v_norm, void* status,
                           cudaStream_t stream);
int pg_softcap(const void* x, void* y, long long n, float cap, cudaStream_t stream);

int pg_repack_int4_pairs(const void* in, void* out, long long words, cudaStream_t stream);

// ---- prefill attention on tcgen05 (attention_tc.cu) ----------------------------------------
int pg_prefill_attention_tc(const void* q, const void* kv_layer, void* out, const void* q_indptr, const void* kv_lens, const void* table, int table_stride,
                            int num_seqs, int tokens, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int q_tiles, void* status,
                            cudaStream_t stream);
void pg_prefill_attention_tc_variant(int v);

// ---- block-scaled FP8 GEMM on tcgen05 kind::f8f6f4 (gemm_fp8_sm100.cu) --------------------
long long pg_gemm_fp8_ws_bytes(int T, int M);
int pg_gemm_fp8_block(const void* xq, long long ldx, const void* x_scale, long long ldxs, const void* wq, long long ldw, const void* w_scale, void* y,
                      long long ldy, int T, int M, int K, void* ws, long long ws_bytes, void* status, cudaStream_t stream);
int pg_quant_fp8_1x128(const void* x, long long ldx, int T, int K, void* xq, long long ldq, void* scale, long long lds, cudaStream_t stream);

int pg_moe_grouped_gemm_fp8(const void* xq, long long rows, const void* x_scale, long long ldxs, const void* wq, const void* w_scale, void* y, long long ldy,
                            const void* offsets, int E, int M, int K, int bn, void* status, cudaStream_t stream);

// ---- sparse-attention indexer (dsa.cu) ----------------------------------------------------
int pg_dsa_k_append(const void* k, long long ld, const void* norm_w, const void* norm_b, const void* cos, const void* sin, const void* positions,
                    const void* slots, void* cache, int tokens, int d, int rope, int max_pos, long long num_slots, float eps, void* status,
                    cudaStream_t stream);
int pg_dsa_q_rope(void* q, const void* cos, const void* sin, const void* positions, int tokens, int heads, int d, int rope, int max_pos, cudaStream_t stream);
int pg_dsa_scores(const void* q, const void* w, const void* cache, const void* unit_seq, const void* q_indptr, const void* kv_lens, const void* table,
                  int table_stride, int page_size, long long num_pages, int tokens, int heads, int d, void* scores, int width, void* status,
                  cudaStream_t stream);
int pg_dsa_topk(const void* scores, int rows, int width, int k, void* out, void* counts, cudaStream_t stream);
int pg_dsa_gather(const void* latent, const void* select, int k, const void* unit_seq, const void* table, int table_stride, int page_size,
                  long long num_pages, int row_bytes, int rows, void* out, int slots_per_row, void* status, cudaStream_t stream);

// ---- multi-head latent attention (mla.cu) ------------------------------------------
int pg_mla_append(const void* kv_a, long long ld, const void* norm_w, const void* cos, const void* sin, const void* positions, const void* slots,
                  void* latent, int tokens, int c, int rope, int max_pos, long long num_slots, float eps, void* status, cudaStream_t stream);
int pg_mla_q_prep(const void* q, const void* cos, const void* sin, const void* positions, void* q_nope_hm, void* q_pe, int tokens, int heads,
                  int nope, int rope, int max_pos, cudaStream_t stream);
int pg_permute_021(const void* in, void* out, int A, int B, int D, cudaStream_t stream);
int pg_mla_attention(const void* q_abs, const void* q_pe, const void* latent, void* out, const void* q_indptr, const void* kv_lens,
                     const void* table, int table_stride, const void* unit_seq, int num_seqs, int tokens, int heads, int c, int rope,
                     int page_size, float scale, int splits, void* part_o, void* part_lse, void* status, cudaStream_t stream);

// ---- mixture of experts (moe_route.cu, moe_gemm.cu) --------------------------------
int pg_router_topk(const void* logits, long long ld, const void* bias, void* ids, void* weights, int tokens, int E, int k, int sigmoid, int n_group,
                   int topk_group, int norm, float scale, cudaStream_t stream);
int pg_moe_align(const void* ids, int routes, int e0, int e_local, void* offsets, void* sorted_src, void* route_pos, cudaStream_t stream);
int pg_moe_gather(const void* x, long long ldx, const void* sorted_src, const void* offsets, int e_local, int k, void* out, int width, int max_rows,
                  cudaStream_t stream);
int pg_moe_combine(const void* y, long long ldy, const void* route_pos, const void* weights, int tokens, int k, void* out, int width, int accumulate,
                   cudaStream_t stream);
// quant: 0 = bf16 weights, 1 = packed INT4 group-32 (+ bf16 scales), 2 = FP8 e4m3 (+ f32 scale_inv per 128x128 block)
int pg_moe_grouped_gemm(const void* x, long long ldx, long long x_rows, const void* w, const void* scales, int quant, void* y, long long ldy,
                        const void* offsets, int E, int M, int K, int bn, void* status, cudaStream_t stream);

int pg_moe_grouped_gemm_return(const void* x, long long ldx, long long x_rows, const void* w, const void* scales, int quant, long long ldy,
                               const void* offsets, int E, int M, int K, int bn, void* status, const void* scatter_src, void* const* peer_out,
                               void* const* peer_flags, int cap, int rank, int world, int site, cudaStream_t stream);
// ---- expert-parallel dispatch / combine over peer memory (ep.cu) -------------------
int pg_ep_dispatch(const void* x, long long ldx, const void* ids, int tokens, const void* valid_tokens, int k, int hidden, int e_local, int cap,
                   void* const* slab, void* const* recv_ids, void* const* flags, int rank, int world, int site, unsigned long long wait_ns,
                   cudaStream_t stream);
int pg_ep_align(const void* recv_ids, int world, int cap, int live, int e_local, void* offsets, void* sorted_src, const void* site_flags,
                unsigned long long wait_ns, void* status, cudaStream_t stream);
int pg_ep_combine(const void* comb, const void* ids, const void* weights, int tokens, int k, void* out, int hidden, const void* valid_tokens,
                  void* site_flags, int world, unsigned long long wait_ns, void* status, cudaStream_t stream);

// ---- LoRA (lora.cu) -----------------------------------------------------------------
int pg_lora_delta(const void* x, long long ldx, const void* A, const void* B, const void* scale, const void* slots, void* y, long long ldy,
                  int tokens, int K, int M, int r_max, int num_slots, void* tvec, cudaStream_t stream);

// ---- Gated DeltaNet (gdn.cu) ------------------------------------------------------
int pg_gdn_conv1d(const void* x, long long ldx, const void* w, void* state, void* out, long long ldo, const void* q_indptr, const void* slots,
                  int num_seqs, int channels, int K, long long state_slot_stride, cudaStream_t stream);
int pg_gdn_gates(const void* a, long long lda, const void* b, long long ldb, const void* a_log, const void* dt_bias, void* g, void* beta,
                 int tokens, int hv, cudaStream_t stream);
int pg_gdn_recurrent(const void* q, const void* k, long long ld_qk, const void* v, long long ld_v, const void* g, const void* beta, void* state,
                     void* out, const void* q_indptr, const void* slots, int num_seqs, int hk, int hv, int dk, int dv, int max_q_len,
                     int skip_len, cudaStream_t stream);
// ---- KDA + attention residuals (kda.cu) ---------------------------------------------
// Delta rule with one decay per key channel; q, k, v share the row stride ld; f [T, heads * dk] and b [T, heads] are the raw
// gate projections (the decay and beta arithmetic runs in the kernel); state [slots, heads, dk, dv] f32.
int pg_kda_recurrent(const void* q, const void* k, const void* v, long long ld, const void* f, long long ldf, const void* b, long long ldb,
                     const void* a_log, const void* dt_bias, float lower, void* state, void* out, const void* q_indptr, const void* slots,
                     int num_seqs, int heads, int dk, int dv, int max_q_len, cudaStream_t stream);
// Softmax mix of the first nb snapshot rows of each token (snaps [T, cap, hidden], ld_tok = cap * hidden) and its current row.
int pg_attnres_mix(const void* cur, long long ld_cur, const void* snaps, long long ld_tok, const void* score_w, void* out, long long ld_out,
                   int tokens, int nb, int hidden, float eps, cudaStream_t stream);
// Chunk-wise (64-token) tensor-core form of the same rule for sequences of >= min_len tokens (gdn_chunk.cu).
int pg_gdn_chunked(const void* q, const void* k, long long ld_qk, const void* v, long long ld_v, const void* g, const void* beta, void* state,
                   void* out, const void* q_indptr, const void* slots, int num_seqs, int hk, int hv, int dk, int dv, int min_len,
                   cudaStream_t stream);

// ---- attention (attention.cu) ------------------------------------------------------
int pg_decode_splits(int num_seqs, int hkv, int max_kv_len, int sms);
void pg_attn_set_decode_stages(int stages);  // 2 (three CTAs per SM) or 3 (two CTAs per SM, default)
int pg_paged_attention(const void* q, const void* kv, void* out, const void* q_indptr, const void* kv_lens, const void* table, int table_stride,
                       int num_seqs, int hq, int hkv, int dim, int page_size, long long num_pages, float scale, int mode, int splits,
                       void* part_o, void* part_lse, int q_tiles, int window, void* status, cudaStream_t stream);

// ---- sampling (sampling.cu) --------------------------------------------------------
long long pg_argmax_scratch_bytes(int rows, int vocab);
int pg_argmax(const void* logits, int is_f32, int rows, int vocab, long long ld, void* scratch, long long scratch_bytes, void* out,
              cudaStream_t stream);
int pg_sample(const void* logits, int is_f32, int rows, int vocab, long long ld, const void* temperature, const void* top_k, const void* top_p,
              const void* min_p, const void* uniform, void* out, cudaStream_t stream);
int pg_logprob_topk(const void* logits, int is_f32, int rows, int vocab, long long ld, const void* picked, int k, void* chosen_lp, void* top_lp,
                    void* top_idx, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
