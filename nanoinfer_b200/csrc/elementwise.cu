// Embedding (+ learned positions), LayerNorm (with an optional row gather) and the
// append of new keys and values to the paged cache.
//
// Formulas: x[t] = wte[tok_t] + wpe[pos_t] (reference: crates/core/src/kernels/reference.rs:86-94);
// LayerNorm two-pass with biased variance, rstd = 1/sqrt(var + eps) (reference.rs:42-51);
// K/V rows of the fused qkv buffer copied to the cache slot of their position
// (crates/core/src/stages/kv_cache.rs:44-57, crates/metal/src/shaders/batch.metal:329-344).
#include "api.h"
#include "common.cuh"

namespace nib {

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                             const T* __restrict__ table, const T* __restrict__ pos_table,
                             float* __restrict__ out, int C) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const T* te = table + (size_t)tokens[t] * C;
  float* o = out + (size_t)t * C;
  if (pos_table != nullptr) {
    const T* pe = pos_table + (size_t)positions[t] * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = to_float(te[c]) + to_float(pe[c]);
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = to_float(te[c]);
  }
}

// ------------------------------------------------------------------ layernorm
// One block per output row.  The row is staged in shared memory as 32-bit floats,
// so the mean and the variance are two true passes over the same values.
template <typename OutT>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 OutT* __restrict__ out, int C, float eps) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;          // C floats
  float* scratch = smem + C;  // 32 floats
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * C;
  float s = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = src[c];
    row[c] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)C;
  float q = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float d = row[c] - mean;
    q += d * d;
  }
  const float var = block_sum(q, scratch) / (float)C;
  const float rstd = 1.0f / sqrtf(var + eps);
  OutT* o = out + (size_t)r * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    o[c] = from_float<OutT>((row[c] - mean) * rstd * gamma[c] + beta[c]);
}

// ------------------------------------------------------------------ kv append
// src is the fused projection output [T, ld]; keys start at column k_off, values at v_off.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ src, int ld, int k_off, int v_off,
                                 T* __restrict__ cache, const int* __restrict__ block_table,
                                 int max_blocks, const int* __restrict__ row_entry,
                                 const int* __restrict__ positions, int n_kv_head, int head_dim,
                                 int page_size, int n_pages, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int page = block_table[(size_t)row_entry[t] * max_blocks + pos / page_size];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) *status = NIB_STATUS_BAD_PAGE;
    return;
  }
  const int slot = pos % page_size;
  const int kv_dim = n_kv_head * head_dim;
  for (int i = threadIdx.x; i < 2 * kv_dim; i += blockDim.x) {
    const int kv = i / kv_dim, rem = i - kv * kv_dim;
    const int h = rem / head_dim, d = rem - h * head_dim;
    const T v = src[(size_t)t * ld + (kv ? v_off : k_off) + rem];
    cache[kv_offset(page, kv, h, slot, n_kv_head, page_size, head_dim) + d] = v;
  }
}

}  // namespace nib

using namespace nib;

extern "C" int nib_embed(int dtype, const int* tokens, const int* positions, const void* table,
                         const void* pos_table, float* out, int T, int C, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = C >= 256 ? 256 : 128;
  if (dtype == DT_F32)
    launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, tokens, positions, (const float*)table,
                                                   (const float*)pos_table, out, C);
  else if (dtype == DT_BF16)
    launch_pdl(embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, tokens, positions, (const bf16*)table,
                                                  (const bf16*)pos_table, out, C);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                             const float* beta, void* out, int n_rows, int C, float eps,
                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const int threads = C >= 1024 ? 512 : (C >= 256 ? 256 : 128);
  if (out_dtype == DT_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, (float*)out, C, eps);
  } else if (out_dtype == DT_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(layernorm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, (bf16*)out, C, eps);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_kv_append(int dtype, const void* src, int ld, int k_off, int v_off, void* cache,
                             const int* block_table, int max_blocks, const int* row_entry,
                             const int* positions, int T, int n_kv_head, int head_dim,
                             int page_size, int n_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = 128;
  if (dtype == DT_F32)
    launch_pdl(kv_append_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)src, ld, k_off, v_off, (float*)cache,
                                                       block_table, max_blocks, row_entry, positions,
                                                       n_kv_head, head_dim, page_size, n_pages, status);
  else if (dtype == DT_BF16)
    launch_pdl(kv_append_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)src, ld, k_off, v_off, (bf16*)cache,
                                                      block_table, max_blocks, row_entry, positions,
                                                      n_kv_head, head_dim, page_size, n_pages, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
