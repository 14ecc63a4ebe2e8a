/* Descriptor of one launch of the fused decode kernel (decode_fused.cu).
 *
 * A launch runs up to four dependent weight-streaming GEMM phases of a decoder layer inside ONE
 * persistent kernel (one CTA per SM): e.g. o-projection -> gate/up -> down -> next layer's q/k/v.
 * Every phase is Y[t, n] = sum_k X[t, k] * W[n, k] with block-scaled FP8 operands (E4M3, fp32 scale
 * per 128-wide K block; weights [n, k] with scales [k/128, ld_sa], activations [rows, k] with scales
 * [k/128, ld_sb]) followed by a fused epilogue that produces the next phase's operand:
 *
 *   PLAIN        y = acc (* norm) (+ residual) (-> soft-cap), bf16 [rows, ldy]
 *   RESID_QUANT  h = acc + residual -> y (bf16, may alias residual), E4M3 + scales of h, and the
 *                per-(128-column block, row) sums of squares of h (for the next RMSNorm)
 *   SILU_QUANT   gate = acc of weight rows [0, n), up = acc of rows [dual_off, dual_off + n):
 *                act(gate * norm) * (up * norm) -> E4M3 + scales
 *   ROPE_KV      one 128-row tile = one attention head: rotate q / k heads, write q (bf16),
 *                quantise k / v heads into their KV page slots
 *
 * "norm": when norm_tiles > 0 the result of row t is multiplied by
 * rsqrt(sum_{i < norm_tiles} ssq_in[i * ld_sb_norm + t] / norm_dim + eps): the RMSNorm in front of the GEMM
 * with its weight vector folded into the weight matrix, applied after the product (the scale is per
 * row, so it commutes with the GEMM).
 *
 * No counterpart in the reference: its decoder layer is one kernel per op
 * (crates/sllm-core/src/qwen_graph.rs:2524-3501).
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

enum { SLLM_FD_MAX_PHASES = 4 };
enum SllmFdEpilogue { SLLM_FD_PLAIN = 0, SLLM_FD_RESID_QUANT = 1, SLLM_FD_SILU_QUANT = 2, SLLM_FD_ROPE_KV = 3 };

typedef struct SllmFdPhase {
  int epilogue;      /* SllmFdEpilogue */
  int n;             /* outputs per row (for SILU_QUANT: the gated width; the weight has dual_off + n rows) */
  int k;             /* reduction length, a multiple of 128 */
  int dual_off;      /* SILU_QUANT: row offset of the "up" half inside the weight; 0 otherwise */
  int norm_tiles;    /* 0: no norm factor */
  int norm_dim;
  int act;           /* SILU_QUANT: 0 SiLU, 1 GELU(tanh) */
  int ldy;           /* row stride of y / residual in elements */
  float eps;
  float softcap;     /* PLAIN: > 0 applies softcap * tanh(y / softcap) */
  int ld_sa;         /* leading dimension of w_scale */
  int ld_sb;         /* leading dimension of x_scale (>= the token tile: 16 or 32) */
  int ld_s_out;      /* leading dimension of s_out / ssq_out / ssq_in */
  int reserved;
  const void* w;     /* E4M3 [rows_w, k] */
  const float* w_scale;
  const void* x;     /* E4M3 [rows, k] */
  const float* x_scale;
  const float* ssq_in;
  void* y;
  const void* residual;
  void* q_out;       /* E4M3 [rows, n] */
  float* s_out;      /* [n / 128, ld_s_out] */
  float* ssq_out;    /* [n / 128, ld_s_out] */
} SllmFdPhase;

typedef struct SllmFdRope {
  const int* positions;    /* [rows] */
  const int* seq_index;    /* [rows] row of block_table owning each token */
  const int* block_table;  /* [seqs, max_blocks] */
  int max_blocks;
  int hq, hkv, rotary_dim, page_size, kv_fp8;
  float theta, k_static, v_static;
  int reserved;
  void* k_pages;           /* [pages, hkv, page, 128] */
  void* v_pages;
  float* k_scale;          /* [pages, hkv, page] (dynamic FP8 only) */
  float* v_scale;
  const float* inv_freq;   /* [rotary_dim / 2] rotary frequencies theta^(-2 i / rotary_dim) (or a scaled variant);
                              read in the kernel preamble: written before the launch is enqueued, by no kernel */
} SllmFdRope;

typedef struct SllmFdDesc {
  int n_phases;
  int rows;                /* tokens (1..32) */
  int n_counters;
  int grid;                /* 0: one CTA per SM */
  SllmFdPhase phase[SLLM_FD_MAX_PHASES];
  SllmFdRope rope;
  float* ws;               /* stream-K partials */
  long long ws_floats;
  int* counters;           /* zero before the first launch; left zero */
  unsigned long long* sync;/* [1] grid-barrier counter, zero before the first launch */
  int* status;
  const void* comm;        /* SllmCommDesc* (host) for RESID_QUANT phases summed across ranks, or null */
  long long wait_limit_cycles;  /* 0: library default */
} SllmFdDesc;

/* Launches the kernel; returns an SllmStatus.  Nothing is allocated. */
int sllm_fused_decode(const SllmFdDesc* desc, void* stream);
/* Workspace floats / counters a launch with this many CTAs needs. */
long long sllm_fused_decode_ws_floats(int grid);
/* Embedding gather producing the operands of the first q/k/v phase: h (bf16), its E4M3 form + scales and the
   per-block sums of squares.  d must be a multiple of 128. */
int sllm_embed_quant(const void* table, const int* ids, void* h, void* q_out, float* s_out, float* ssq_out, int ld_s,
                     int rows, int d, int vocab, float scale, void* stream);
/* Profiling aid: device buffer of [CTAs][4][8] 64-bit words that later launches fill with globaltimer stamps per phase
   (0 set-up done, 1 phase input visible, 2 first accumulator ready, 3 last segment promoted, 4 last tile complete,
   5 outputs written, 6 arrived at the grid barrier); null switches it off. */
void sllm_fused_decode_set_trace(void* dev_buf);
/* Tuning knob: L2 prefetch distance of the weight producer, in 16 KB tiles per CTA (0 = none). */
void sllm_fused_decode_set_lookahead(int tiles);
/* sizeof / offsetof records of the descriptor structs for a layout check by foreign-language bindings:
   writes up to n ints, returns how many the library has. */
int sllm_fused_decode_abi(int* out, int n);

#ifdef __cplusplus
}
#endif
