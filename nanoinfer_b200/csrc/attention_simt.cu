// General causal attention over the paged cache: one warp per (query row, head).
//
// It takes any mix of rows (prompt portions and single decoded tokens), any head
// size up to 256, any number of heads and key/value heads, and an optional window.
// Formula (reference: crates/core/src/kernels/reference.rs:109-142): s_j = (q . k_j) * scale
// for the keys j <= pos, softmax with the maximum subtracted, o = sum_j p_j v_j.  The
// softmax runs online over blocks of 32 keys (the split/merge rule of
// crates/metal/src/shaders/batch.metal:349-424), all in 32-bit.  A row's result depends on
// its own keys only, never on what else the batch holds.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_ND = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* q, int ldq, const T* cache,
                      T* out, int ldo, const int* __restrict__ block_table,
                      int max_blocks, const int* __restrict__ rows, const int* __restrict__ row_entry,
                      const int* __restrict__ positions, int n_head, int n_kv_head, int head_dim,
                      int page_size, int n_pages, float scale, int window, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * ATT_WARPS + warp;
  const int t = rows ? rows[blockIdx.y] : blockIdx.y;
  if (h >= n_head) return;  // whole warps leave; no block-wide barrier follows
  if (row_entry[t] < 0) return;   // a row of no request (padding): nothing to attend to
  float* qs = smem + (size_t)warp * (head_dim + 32 + 64);
  float* pj = qs + head_dim;                                   // 32 probabilities
  unsigned long long* voff = (unsigned long long*)(pj + 32);   // 32 value-row offsets (8-byte aligned)

  const int pos = positions[t];
  const int* table = block_table + (size_t)row_entry[t] * max_blocks;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int hk = h / (n_head / n_kv_head);

  for (int d = lane; d < head_dim; d += 32) qs[d] = to_float(q[(size_t)t * ldq + h * head_dim + d]);
  __syncwarp();

  float o[ATT_MAX_ND];
#pragma unroll
  for (int i = 0; i < ATT_MAX_ND; ++i) o[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;

  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= pos;
    float s = -INFINITY;
    unsigned long long vo = 0;
    if (valid) {
      const int page = table[j / page_size];
      if (page < 0 || page >= n_pages) {
        *status = NIB_STATUS_BAD_PAGE;
      } else {
        const int slot = j % page_size;
        const T* kr = cache + kv_offset(page, 0, hk, slot, n_kv_head, page_size, head_dim);
        vo = kv_offset(page, 1, hk, slot, n_kv_head, page_size, head_dim);
        float dot = 0.0f;
        for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAX_ND; ++i) o[i] *= corr;
    pj[lane] = p;
    voff[lane] = vo;
    __syncwarp();
    const int n_valid = min(32, pos - j0 + 1);
    for (int jj = 0; jj < n_valid; ++jj) {
      const float pv = pj[jj];
      const T* vr = cache + voff[jj];
#pragma unroll
      for (int i = 0; i < ATT_MAX_ND; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) o[i] = fmaf(pv, to_float(vr[d]), o[i]);
      }
    }
    __syncwarp();
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < ATT_MAX_ND; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) out[(size_t)t * ldo + h * head_dim + d] = from_float<T>(o[i] * inv);
  }
}

}  // namespace nib

using namespace nib;

extern "C" int nib_attention_simt(int dtype, const void* q, int ldq, const void* cache, void* out,
                                  int ldo, const int* block_table, int max_blocks, const int* rows,
                                  const int* row_entry, const int* positions, int T, int n_head,
                                  int n_kv_head, int head_dim, int page_size, int n_pages,
                                  float scale, int window, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (head_dim <= 0 || head_dim > 32 * ATT_MAX_ND || (head_dim & 1)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0) return NIB_ERR_BAD_ARGUMENT;
  if (T > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  dim3 grid((n_head + ATT_WARPS - 1) / ATT_WARPS, T);
  const size_t smem = (size_t)ATT_WARPS * (head_dim + 32 + 64) * sizeof(float);
  if (dtype == DT_F32)
    launch_pdl(attention_simt_kernel<float>, dim3(grid), dim3(ATT_WARPS * 32), smem, stream, 
        (const float*)q, ldq, (const float*)cache, (float*)out, ldo, block_table, max_blocks, rows, row_entry,
        positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, status);
  else if (dtype == DT_BF16)
    launch_pdl(attention_simt_kernel<bf16>, dim3(grid), dim3(ATT_WARPS * 32), smem, stream, 
        (const bf16*)q, ldq, (const bf16*)cache, (bf16*)out, ldo, block_table, max_blocks, rows, row_entry,
        positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
