/* C ABI of the sm_100a kernel library (libsllm_b200_kernels.so).
 *
 * Conventions shared by every entry point:
 *   - returns 0 when the kernel was launched, a small positive SllmStatus code otherwise; nothing is
 *     launched when arguments are rejected;
 *   - pointers are device pointers unless the name says otherwise; `stream` is a cudaStream_t;
 *   - no compute entry point allocates device memory: workspaces and counters are supplied by the
 *     caller (counters must be zero before the first launch; kernels leave them zero); only
 *     sllm_symm_alloc / sllm_symm_open create or map device memory;
 *   - kernels that wait on barriers write a non-zero code to `status` (device int) instead of hanging.
 *
 * The role of this header mirrors the reference's include/sllm/hip.h (status codes :27-85, one
 * prepare/execute pair per op :1274-1692), collapsed to one validated launch call per op.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

/* gemm_tcgen05.cu */
long long sllm_gemm_workspace_floats(int a_rows, int b_rows, int bn, int splits);
int sllm_gemm(const void* a, const void* b, void* y, const float* scale_a, const float* scale_b,
              const void* residual, int a_rows, int b_rows, int k, int scaled, int transpose_out, int ldy,
              int ld_sa, int ld_sb, int bn, int splits, int stages, float* ws, long long ws_floats, int* counters,
              int n_counters, int* status, void* stream);

void sllm_gemm_set_cluster_split(int enabled);
int sllm_gemm_allreduce(const void* a, const void* b, void* y, const float* scale_a, const float* scale_b,
                        const void* residual, int a_rows, int b_rows, int k, int scaled, int transpose_out, int ldy,
                        int ld_sa, int ld_sb, int bn, int splits, int stages, float* ws, long long ws_floats,
                        int* counters, int n_counters, int* status, void* stream, const void* comm);

/* elementwise.cu */
int sllm_embedding(const void* table, const int* ids, void* out, int tokens, int d, int vocab, float scale,
                   void* stream);
int sllm_rmsnorm(const void* x, const void* w, void* y_bf16, void* y_fp8, float* y_scale, int ld_scale, int rows,
                 int d, float eps, int offset_one, void* stream);
int sllm_gated_act(const void* in, void* y_bf16, void* y_fp8, float* y_scale, int ld_scale, int rows, int inter,
                   int act, void* stream);
int sllm_quant_fp8_1x128(const void* x, void* y, float* scale, int ld_scale, int rows, int k, void* stream);
int sllm_rope_kv_append(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                        int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale, int tokens,
                        int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8, float theta,
                        float k_static_scale, float v_static_scale, const float* inv_freq, void* stream);
/* rope_pos3 [3, tokens]: temporal / height / width rotary index per token; rotary pair j uses axis 0 for
   j < sec_t, axis 1 for j < sec_t + sec_h, axis 2 otherwise.  The page slot still comes from positions. */
int sllm_rope_kv_append_mrope(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                              int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale, int tokens,
                              int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8, float theta,
                              float k_static_scale, float v_static_scale, const float* inv_freq,
                              const int* rope_pos3, int sec_t, int sec_h, void* stream);
/* pair_offset > 0: channel i < rotary_dim / 2 pairs with i + pair_offset and frequencies are theta^(-2 i / hd). */
int sllm_rope_kv_append_paired(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                               int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale, int tokens,
                               int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8, float theta,
                               float k_static_scale, float v_static_scale, const float* inv_freq, int pair_offset,
                               void* stream);
int sllm_elementwise(const void* a, const void* b, void* y, long long n, int d, int op, float s, void* stream);
int sllm_argmax(const void* logits, int* out_idx, float* out_val, int rows, int n, int ld, int index_offset,
                void* ws, long long ws_bytes, int* counters, int n_counters, void* stream);

/* attention.cu */
long long sllm_paged_attention_workspace_floats(int rows, int hq, int hd, int hkv, int splits);
int sllm_paged_attention(const void* q, int q_ld, const void* k_pages, const void* v_pages, const float* k_scale,
                         const float* v_scale, float k_static_scale, float v_static_scale, const int* block_table,
                         int max_blocks, const int* seq_index, const int* kv_lens, int rows, int hq, int hkv, int hd,
                         int page_size, int window, float sm_scale, int kv_fp8, void* out_bf16, void* out_fp8,
                         float* out_scale, int ld_scale, const float* sinks, int splits, float* ws,
                         long long ws_floats, int* counters, int n_counters, void* stream);

/* decode_attention_tc.cu */
int sllm_decode_attention_tc(const void* q, int q_ld, const void* k_pages, const void* v_pages, const float* k_scale,
                             const float* v_scale, float k_static_scale, float v_static_scale,
                             const int* block_table, int max_blocks, const int* seq_index, const int* kv_lens,
                             int rows, int hq, int hkv, int num_pages, int page_size, int window, float sm_scale,
                             void* out_bf16, void* out_fp8, float* out_scale, int ld_scale, const float* sinks,
                             int splits, float* ws, long long ws_floats, int* counters, int n_counters, int* status,
                             void* stream);

/* prefill_attention.cu */
int sllm_prefill_attention(const void* qkv, int total_tokens, int qkv_ld, const int* tiles, int num_tiles, int hq,
                           int hkv, int hd, float sm_scale, void* out_bf16, void* out_fp8, float* out_scale,
                           int ld_scale, int* status, void* stream);

/* comm.cu */
int sllm_symm_alloc(long long bytes, void** dev_ptr, unsigned char* handle64);
int sllm_symm_open(const unsigned char* handle64, void** dev_ptr);
int sllm_symm_close(void* peer_ptr);
int sllm_symm_free(void* dev_ptr);
int sllm_allgather_small(const void* const* bases, int world, int rank, long long offset, long long flag_offset,
                         int slot_bytes, const void* src, void* dst, void* epoch, int* status, void* stream);
int sllm_argmax_merge(const float* vals, const int* idx, int* out, int rows, int world, void* stream);

#ifdef __cplusplus
}
#endif
