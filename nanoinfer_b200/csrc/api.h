// C interface of the kernel library.  Every launcher enqueues on `stream`, allocates
// nothing, and returns 0 or an error code: a positive value is a cudaError_t, a
// negative one is one of the NIB_ERR_* codes below.
#pragma once

#include <cuda_runtime.h>

#define NIB_ERR_BAD_ARGUMENT (-1)
#define NIB_ERR_UNSUPPORTED_SIZE (-2)
#define NIB_ERR_DRIVER (-3)

// Values a kernel may leave in the device status word.
#define NIB_STATUS_OK 0
#define NIB_STATUS_BAD_PAGE 1
#define NIB_STATUS_WAIT_TIMEOUT 2

#ifdef __cplusplus
extern "C" {
#endif

// A negative token -(s + 1) stands for feedback[s]: the token that the step before sampled for
// slot s and left on the device (feedback may be null when no token is negative).
int nib_embed(int dtype, const int* tokens, const int* positions, const void* table,
              const void* pos_table, const int* feedback, float* out, int T, int C, cudaStream_t stream);

int nib_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                  const float* beta, void* out, int n_rows, int C, float eps, cudaStream_t stream);

int nib_kv_append(int dtype, const void* src, int ld, int k_off, int v_off, void* cache,
                  const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                  int T, int n_kv_head, int head_dim, int page_size, int n_pages, int* status,
                  cudaStream_t stream);

// out[M,N] = act(a[M,K] . w[N,K]^T + bias); with `residual` the result is added to the
// 32-bit `out` in place.  SIMT path: true 32-bit arithmetic for float inputs.
int nib_linear_simt(int in_dtype, int out_dtype, const void* a, int lda, const void* w, int ldw,
                    const float* bias, void* out, int ldo, int M, int N, int K, int act,
                    int residual, cudaStream_t stream);

// The same product for bfloat16 inputs on the tensor cores (tcgen05 + TMA); out is bfloat16 or
// float32.  nib_linear_tc_supported says whether the shape and alignment are taken.
int nib_linear_tc_supported(const void* a, int lda, const void* w, int ldw, int K);
int nib_linear_tc(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                  void* out, int ldo, int M, int N, int K, int act, int residual, int* status,
                  cudaStream_t stream);

// The general tensor-core product for steps of at most 128 rows, with three options: activations made
// in the kernel by LayerNorm of the 32-bit residual stream (ln_x), keys and values written straight
// into a cache layer (cache), and K split over blocks through caller-provided scratch
// (fix_partials / fix_counters; the counters are zero before the first call and left zero).
int nib_linear_tc_small(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                        void* out, int ldo, int M, int N, int K, int act, int residual, const float* ln_x,
                        int ln_ldx, const float* ln_gamma, const float* ln_beta, float ln_eps,
                        const int* ln_rows, void* cache, const int* block_table, int max_blocks,
                        const int* row_entry, const int* positions, int q_dim, int n_kv_head, int head_dim,
                        int page_size, int n_pages, float* fix_partials, long long fix_floats,
                        int* fix_counters, int fix_n_counters, int* status, cudaStream_t stream);

// The product for many rows by pairs of blocks that share one 256-row MMA (cta_group::2): each block
// loads its own 128 rows of the activations and half of the weight tile.  bq: columns of a tile (0:
// chosen by the library; else a multiple of 32 up to 256); splits: splits of K for residual outputs
// (0: chosen by the library).  cache != null: the fused q/k/v projection, keys and values straight
// into the rows' slots of one cache layer (q_dim a multiple of 64, head_dim of 16).
int nib_linear_tc_pair_supported(int out_dtype, const void* a, int lda, const void* w, int ldw, const void* out,
                                 int ldo, int M, int N, int K, int residual);
int nib_linear_tc_pair(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                       int ldo, int M, int N, int K, int act, int residual, int bq, int splits, void* cache,
                       const int* block_table, int max_blocks, const int* row_entry, const int* positions,
                       int q_dim, int n_kv_head, int head_dim, int page_size, int n_pages, int* status,
                       cudaStream_t stream);

// The product for steps of at most 128 rows with warp-level MMAs (bfloat16; row blocks of 16), with the same
// LayerNorm and cache options as nib_linear_tc_small.  split: blocks of a cluster that split
// K (0: chosen by the library; else 1, 2, 4 or 8).
int nib_linear_skinny_supported(int M, int K, int ldw, int ln, const void* w);
int nib_linear_skinny(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                      int ldo, int M, int N, int K, int act, int residual, const float* ln_x, int ln_ldx,
                      const float* ln_gamma, const float* ln_beta, float ln_eps, const int* ln_rows,
                      void* cache, const int* block_table, int max_blocks, const int* row_entry,
                      const int* positions, int q_dim, int n_kv_head, int head_dim, int page_size, int n_pages,
                      int split, int* status, cudaStream_t stream);

// Causal attention of T query rows over the paged cache (general SIMT kernel).  rows: the
// step's rows to process (nullptr: rows 0..T-1).
int nib_attention_simt(int dtype, const void* q, int ldq, const void* cache, void* out, int ldo,
                       const int* block_table, int max_blocks, const int* rows, const int* row_entry,
                       const int* positions, int T, int n_head, int n_kv_head, int head_dim,
                       int page_size, int n_pages, float scale, int window, int* status,
                       cudaStream_t stream);

// tcgen05 attention for prompt portions (bfloat16, head size 64, page size a multiple of 16): tiles of
// 128 query rows, S and O in tensor memory, keys and values by TMA page by page.  q holds T rows.
int nib_attention_prefill_tc_supported(int head_dim, int page_size);
int nib_attention_prefill_tc(const void* q, int ldq, int T, const void* cache, void* out, int ldo,
                             const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                             const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head, int head_dim,
                             int page_size, int n_pages, float scale, int window, int* status, cudaStream_t stream);

// Split-KV attention for single decoded tokens (float32 or bfloat16, head sizes up to 128 in steps
// of 8, pages of a multiple of 16 positions) and its scratch need.
long long nib_attention_decode_scratch(int n_rows, int n_head, int head_dim, int n_splits);
int nib_attention_decode(int dtype, const void* q, int ldq, const void* cache, float* scratch, void* out,
                         int ldo, const int* block_table, int max_blocks, const int* rows,
                         const int* row_entry, const int* positions, int n_rows, int n_head, int n_kv_head,
                         int head_dim, int page_size, int n_pages, float scale, int window, int chunk,
                         int n_splits, int* counters, int* status, cudaStream_t stream);

// Tiled tensor-core attention for prompt portions (bfloat16, head sizes 16..128 in steps of 16).
int nib_attention_prefill_supported(int head_dim);
int nib_attention_prefill(const void* q, int ldq, const void* cache, void* out, int ldo,
                          const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                          const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head,
                          int head_dim, int page_size, int n_pages, float scale, int window, int* status,
                          cudaStream_t stream);

// Loading: src holds [rows, cols] values as a checkpoint stores them (src_dtype 0: 32-bit floats, 1:
// bfloat16, 2: 16-bit floats); element (r, c) is converted to dst_dtype and written to
// dst[(r0 + r) * ld + c], or with `transpose` to dst[c * ld + r0 + r].
int nib_convert(int src_dtype, const void* src, int rows, int cols, int dst_dtype, void* dst, long long ld,
                long long r0, int transpose, cudaStream_t stream);

int nib_argmax(const float* logits, int ld, int n_rows, int V, int* out, cudaStream_t stream);

// One token per logits row.  temperature, top_k and rng_state are per-slot arrays indexed by
// row_slot[r]: argmax where temperature <= 0, else temperature / top-k sampling with the
// request's own xorshift64* state (advanced by one draw).
// last_token (may be null): per-slot array that also receives each row's token, for the next step's
// embedding to read.
// scratch: 2 * n_rows 64-bit words that are zero before the first call (the kernel leaves them zero).
// teams != 0: the launch is made of clusters whose blocks share a sampled row's passes (for steps in
// which some row may be sampled; the tokens are the same either way).
int nib_sample(const float* logits, int ld, int n_rows, int V, const int* row_slot,
               const float* temperature, const int* top_k, unsigned long long* rng_state, int* out,
               int* last_token, unsigned long long* scratch, int teams, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
