// C entry points of libogb200_kernels.so (sm_100a).  Every launcher takes raw device pointers and
// a CUDA stream (void* = cudaStream_t), launches asynchronously and returns 0 on success or a
// negative code: -1 bad argument / alignment, -2 scratch or tensor-map failure, -3 attribute
// failure, -4 launch failure, -5 unsupported shape.  None of them allocates device memory.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- runtime.cu
int ogb_runtime_init(int device);                 // allocates the per-device status word (call outside graph capture)
int* ogb_status_device_ptr(int device);           // device address of the status word
int ogb_status_read_and_clear(int device);        // synchronises the device; returns the OgbStatus code seen since last call
int ogb_sm_count(int device);
const char* ogb_last_cuda_error();

// ---- gemm_tcgen05.cu
int ogb_gemm_token_tile(int M, int dual);
int ogb_gemm_max_active_clusters(int bt, int splits);
int ogb_gemm_auto_splits(int M, int N, int K, int dual, int sm_count);
int ogb_comm_register(int device, int world, int rank, void** buf, void* epoch, long long plane_elems);
int ogb_comm_register_nvls(int device, void* data, void* data_mc, void* out, void* out_mc, void* ctr, void* ctr_mc, void* expected,
                           long long plane_elems);
int ogb_comm_has_nvls(int device);
int ogb_comm_set_options(int use_nvls, long long two_shot_bytes, int p2p_two_hop);   // negative (-2 for the last): leave unchanged
long long ogb_comm_capacity(int device);
// flags: bit 0 fp32 output, bit 1 paired silu(gate)*up epilogue, bit 2 fused tensor-parallel all-reduce,
// bit 3 fused reduce-scatter by token rows (sequence-parallel form)
int ogb_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, const void* bias,
                  const void* residual, int ldr, int flags, int splits, int device, int* status, int sm_count, void* stream);

// Decode-step fusions of ogb_gemm_bf16_fused (all pointers are device pointers).
typedef struct OgbGemmFused {
  float norm_eps;            // > 0: RMS norm folded into the GEMM (row scale rsqrt(mean(x^2) + eps); the weight carries the norm's weight)
  const int32_t* positions;  // != NULL: QKV projection with rotary embedding + KV-cache append in the epilogue
  const int32_t* slots;      // cache row of each token (< 0: not stored)
  const float* cos;          // [max_pos, rot / 2]
  const float* sin;
  void* k_cache;             // bf16 [slots, Hkv, D]
  void* v_cache;
  int Hq, Hkv, D, rot, max_pos;
} OgbGemmFused;
int ogb_gemm_bf16_fused(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, const void* bias,
                        const void* residual, int ldr, int flags, int splits, int device, int* status, int sm_count, void* stream,
                        const OgbGemmFused* fused);

// Grouped expert GEMM over token rows sorted by expert (tile list from ogb_moe_sort); act_kind 1 = silu(gate)*up,
// 2 = clamped SwiGLU(alpha, limit); flags as above (bit 2 unused).
int ogb_moe_gemm(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int rows_total, int N, int K, int experts,
                 const void* bias, int flags, int act_kind, float act_alpha, float act_limit, const int* tile_expert,
                 const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles, int token_tile, int* status,
                 void* stream);

// ---- collectives.cu: mode 0 all-reduce, 1 all-gather, 2 reduce-scatter over the registered symmetric buffers (bf16)
int ogb_collective(int mode, const void* in, void* out, const void* residual, long long n, int device, int* status, int sm_count,
                   void* stream);

// ---- moe.cu
int ogb_moe_topk(const float* logits, int ld, int T, int E, int k, int mode, int32_t* topk_idx, float* topk_w, void* stream);
int ogb_moe_max_tiles(int n, int experts, int bt);
int ogb_moe_fp4_reads_row_map(int token_tile, int K, int half);
int ogb_moe_sort(const int32_t* topk_idx, int T, int k, int E, int e_lo, int e_hi, int bt, int32_t* expert_offsets,
                 int32_t* sorted_token, int32_t* inv_pos, int32_t* tile_expert, int32_t* tile_row0, int32_t* tile_rows,
                 int32_t* num_tiles, int max_tiles, void* stream);
int ogb_moe_combine(const void* y, int ldy, const int32_t* inv_pos, const float* topk_w, int T, int k, int H, const void* residual,
                    int ldr, void* out, int ldo, void* stream);

// ---- gemm_w4.cu (int4 block-32 weights, repacked by ops.pack_w4)
long long ogb_w4_packed_bytes(int N, int K);
int ogb_gemm_w4(const void* A, int lda, const void* Wpacked, void* C, int ldc, int M, int N, int K, const void* bias,
                const void* residual, int ldr, int flags, int splits, int* status, int sm_count, void* stream);

// ---- gemm_fp4.cu (MXFP4 experts kept packed: e2m1 codes + e8m0 block scales, repacked by ops/fp4.py)
long long ogb_fp4_packed_bytes(int experts, int N, int K);
int ogb_moe_gemm_fp4(const void* A, int lda, const void* Wpacked, void* C, int ldc, int rows_total, int N, int K, int experts,
                     const void* bias, int flags, int act_kind, float act_alpha, float act_limit, const int* tile_expert,
                     const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles, int token_tile,
                     int max_rows_per_tile, const int32_t* row_map, int* status, void* stream);

// ---- elementwise.cu
int ogb_embedding(const int32_t* ids, const void* table, void* out, int T, int H, int vocab, float scale, void* stream);
int ogb_norm(const void* x, const void* residual_in, void* residual_out, const void* weight, const void* bias, void* out,
             int rows, int H, float eps, int layernorm, void* stream);
int ogb_norm_moe_combine(const void* y, int ldy, const int32_t* inv_pos, const float* topk_w, int k, const void* residual_in, void* residual_out,
                         const void* weight, const void* bias, void* out, int rows, int H, float eps, int layernorm, void* stream);
int ogb_rope_kv_append(void* qkv, int qkv_stride, const int32_t* positions, const int32_t* slots, const float* cos_cache,
                       const float* sin_cache, void* k_cache, void* v_cache, const void* q_norm_w, const void* k_norm_w,
                       float norm_eps, int T, int Hq, int Hkv, int D, int rot, int interleaved, int max_pos, void* stream);
int ogb_rope_kv_append_bits(void* qkv, int qkv_stride, const int32_t* positions, const int32_t* slots, const float* cos_cache,
                       const float* sin_cache, void* k_cache, void* v_cache, const void* q_norm_w, const void* k_norm_w,
                       float norm_eps, int T, int Hq, int Hkv, int D, int rot, int interleaved, int max_pos, int kv_bits, const int32_t* positions3, int sec0, int sec1, void* stream);
int ogb_embedding_q4(const int32_t* ids, const void* q, const void* scales, const void* zps, void* out, int T, int K, int vocab,
                     float mult, void* stream);
int ogb_act_mul(const void* x, void* out, int T, int I, int act, void* stream);
int ogb_act(const void* x, void* out, long long n, int act, void* stream);
int ogb_causal_conv(const void* x, int x_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                    const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                    int table_cols, int block_size, void* out, int T, int B, int C, int L, int silu, void* stream);
int ogb_short_conv(const void* bcx, int bcx_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                   const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                   int table_cols, int block_size, void* out, int T, int B, int C, int L, void* stream);
int ogb_decode_advance(const int32_t* sampled, int32_t* input_ids, int32_t* positions, int32_t* past_lens, int32_t* slot_mapping,
                       int32_t* sample_pos, const int32_t* block_table, int table_cols, int block_size, int B, void* stream);
int ogb_logits_edit(float* logits, int vocab, const int32_t* rows, const int32_t* tokens, const int32_t* ops,
                    const float* values, int n, void* stream);
int ogb_logits_bitmask(float* logits, int rows, int vocab, const uint32_t* mask, const int32_t* mask_rows, void* stream);
int ogb_bf16_to_f32(const void* in, float* out, long long n, void* stream);
int ogb_gather_rows(const void* in, const int32_t* rows, void* out, int n_rows, int row_bytes, void* stream);
int ogb_gather_rows_f16(const void* in, const int32_t* rows, void* out, int n_rows, int row_bytes, void* stream);  // bf16 -> fp16

// ---- linear_attention.cu: gated delta rule over packed sequences; state [slots, Hv, dk, dv] fp32 updated in place
int ogb_gated_delta_fused(const void* conv, long long conv_stride, long long q_off, long long k_off, long long v_off, const void* ba,
                          long long ba_stride, long long b_off, long long a_off, const float* neg_exp_a, const float* dt_bias, float q_scale,
                          float* state, const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int Hk,
                          int Hv, int dk, int dv, void* stream);
int ogb_gdn_gate_norm(const void* o, const void* z, long long z_stride, const float* w, float eps, void* out, int T, int Hv, int dv, void* stream);
int ogb_gated_delta(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, const int32_t* slots,
                    const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int Hk, int Hv, int dk, int dv, void* stream);
int ogb_mamba2_scan_fused(const void* conv, long long conv_stride, const void* dt_raw, long long dt_stride, const float* dt_bias, const float* neg_a,
                          const float* Dv, float* state, const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B,
                          int heads, int groups, int P, int N, void* stream);
int ogb_mamba_gate_norm(const void* y, const void* z, long long z_stride, const float* w, float eps, void* out, int T, int I, void* stream);
int ogb_mamba2_scan(const void* x, const float* dt, const float* neg_a, const void* Bm, const void* Cm, const float* Dv, float* state,
                    const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int heads, int groups, int P, int N,
                    void* stream);
int ogb_copy_state_slots(const float* src, float* dst, int layers, int slots, long long slot_elems, const int32_t* src_slots,
                         const int32_t* dst_slots, int count, void* stream);

// ---- attention.cu
long long ogb_attention_scratch_bytes(int total_tokens, int Hq, int D, int splits);
// cache_slots (rows of the key / value cache) and status (device status word) enable the TMA-fed K/V path; 0 / null keep
// the cp.async path.  order: optional [B] permutation of the requests in which the CTAs are issued (longest first balances
// a batch of mixed lengths).  splits > 1 divides a request's keys between CTAs: evenly (kv_chunk 0) or in fixed ranges of kv_chunk keys (multiple of 64).
int ogb_paged_attention(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                        const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                        int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                        int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch, long long scratch_bytes,
                        int cache_slots, const int32_t* order, int* status, void* stream);
// attention_tc.cu: tcgen05 prefill attention for the requests of a launch with at least `min_rows` query rows (bf16 cache,
// head_dim 64 / 128, cache blocks of a multiple of 16 tokens); ogb_paged_attention_skip serves the others.
int ogb_attention_tc_supported(int D, int block_size, int kv_bits, int cache_slots);
int ogb_attention_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                     const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out, int out_stride,
                     const float* sinks, float scale, float softcap, int window, int B, int max_q_len, int Hq, int Hkv, int D,
                     int min_rows, int cache_slots, int* status, void* stream);
int ogb_paged_attention_skip(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                             const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                             int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                             int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch,
                             long long scratch_bytes, int cache_slots, const int32_t* order, int* status, void* stream, int skip_rows);
int ogb_paged_attention_kv8(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                        const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                        int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                        int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch, long long scratch_bytes,
                        int cache_slots, const int32_t* order, int* status, void* stream);

// ---- sampling.cu
int ogb_sample(const float* logits, long long row_stride, int rows, int vocab, const int32_t* top_k, const float* top_p,
               const float* temperature, const unsigned long long* seeds, const int32_t* positions, int32_t* out, void* stream);
int ogb_argmax(const float* logits, long long row_stride, int rows, int vocab, int32_t* out, void* stream);
int ogb_topk(const float* x, long long row_stride, int rows, int n, int k, int mode, const float* add, float* out_vals,
             int32_t* out_idx, void* stream);
int ogb_beam_merge(const float* in_vals, const int32_t* in_idx, int batch, int beams, int cand, float* out_scores,
                   int32_t* out_tokens, int32_t* out_beams, void* stream);
// Beam scorer + sequence append on the device (beam_scorer.cu)
int ogb_beam_scorer_step(const float* cand_scores, const int32_t* cand_tokens, const int32_t* cand_beams, void* seq0, void* seq1, int cur, int len,
                         void* scores, void* hyp_tokens, void* hyp_len, void* hyp_score, void* hyp_order, void* hyp_count, void* done, void* out,
                         int batch, int num_beams, int max_length, int pad_token, int early_stopping, float length_penalty, const int32_t* eos,
                         int n_eos, void* stream);
int ogb_beam_scorer_finalize(void* seq0, void* seq1, int cur, int len, void* scores, void* hyp_tokens, void* hyp_len, void* hyp_score,
                             void* hyp_order, void* hyp_count, void* done, void* out, int batch, int num_beams, int max_length, int pad_token,
                             int early_stopping, float length_penalty, const int32_t* eos, int n_eos, void* stream);
int ogb_verify_sampled(const float* logits, long long row_stride, int vocab, int K, const int32_t* top_k, const float* top_p,
                       const float* temperature, const unsigned long long* seeds, const int32_t* positions, const int32_t* draft,
                       const int32_t* q_idx, const float* q_prob, const int32_t* q_n, int q_stride, int32_t* scratch,
                       float* accept_prob, int32_t* accepted, int32_t* commit, int32_t* status, void* stream);
int ogb_verify_greedy(const int32_t* draft, const int32_t* target_argmax, int k, int32_t* accepted, int32_t* commit, void* stream);

#ifdef __cplusplus
}
#endif
