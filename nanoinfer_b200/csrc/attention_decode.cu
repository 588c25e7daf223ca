// Attention for single decoded tokens: split-KV "flash decoding" over the block tables.
//
// One block handles one (row, head, split of the keys): it streams its share of the paged keys
// and values once, keeps an online softmax (running maximum m, sum l, unnormalised output o) and
// writes the partial (m, l, o); a second kernel merges the splits of a (row, head) in a fixed
// order:  M = max m_s;  L = sum l_s e^(m_s - M);  out = sum o_s e^(m_s - M) / L.
// This is the reference's b_attn_split / b_attn_merge pair
// (crates/metal/src/shaders/batch.metal:349-424) with the split size chosen by the host so that
// a small batch still fills the GPU.  Scores are (q . k) * scale for the keys lo..pos, in 32-bit
// (crates/core/src/kernels/reference.rs:109-142).
//
// Inside a block each warp takes 16 keys at a time: two lanes share a key for the dot product
// (each reads alternate 16-byte pieces of the key row), then the lanes turn to the head
// dimensions for the weighted sum of the values.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int DEC_WARPS = 4;
constexpr int DEC_MAX_PAIRS = 4;  // head_dim <= 256: lane owns dims 2*lane + 64*i, +1

template <typename T> struct Vec16;  // one 16-byte piece of a row
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ float dot(const float* __restrict__ k, const float* q) {
    const float4 v = *reinterpret_cast<const float4*>(k);
    return v.x * q[0] + v.y * q[1] + v.z * q[2] + v.w * q[3];
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ float dot(const bf16* __restrict__ k, const float* q) {
    const uint4 raw = *reinterpret_cast<const uint4*>(k);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      s = fmaf(f.x, q[2 * i], s);
      s = fmaf(f.y, q[2 * i + 1], s);
    }
    return s;
  }
};
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// partial layout: o [row][head][split][head_dim], ml [row][head][split][2]
template <typename T>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache, float* __restrict__ part_o,
                        float* __restrict__ part_ml, T* __restrict__ out, int ldo,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ rows,
                        const int* __restrict__ row_entry, const int* __restrict__ positions, int n_head,
                        int n_kv_head, int head_dim, int page_size, int n_pages, float scale, int window,
                        int chunk, int n_splits, int* __restrict__ status) {
  extern __shared__ float smem[];
  float* qs = smem;                                  // head_dim
  float* wo = smem + head_dim;                       // DEC_WARPS * head_dim
  float* wm = wo + DEC_WARPS * head_dim;             // DEC_WARPS
  float* wl = wm + DEC_WARPS;                        // DEC_WARPS
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  const int t = rows ? rows[r] : r;
  const int pos = positions[t];
  const int* table = block_table + (size_t)row_entry[t] * max_blocks;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);  // exclusive
  const int hk = h / (n_head / n_kv_head);
  const size_t pidx = ((size_t)r * n_head + h) * n_splits + split;

  if (k_begin >= k_end) {  // nothing in this split: the merge skips l == 0
    if (threadIdx.x == 0) {
      part_ml[2 * pidx] = -INFINITY;
      part_ml[2 * pidx + 1] = 0.0f;
    }
    return;
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = to_float(q[(size_t)t * ldq + h * head_dim + d]);
  __syncthreads();

  constexpr int VN = Vec16<T>::N;
  const int n_pieces = head_dim / VN;  // 16-byte pieces per key row
  const int key_in_unit = lane >> 1, half = lane & 1;
  float o[2 * DEC_MAX_PAIRS];
#pragma unroll
  for (int i = 0; i < 2 * DEC_MAX_PAIRS; ++i) o[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;

  // units of 16 consecutive keys that lie in one page (page_size is a multiple of 16)
  const int first_unit = k_begin / 16, last_unit = (k_end - 1) / 16;
  for (int u = first_unit + warp; u <= last_unit; u += DEC_WARPS) {
    const int j0 = u * 16;
    const int page = table[j0 / page_size];
    if (page < 0 || page >= n_pages) {
      if (lane == 0) *status = NIB_STATUS_BAD_PAGE;
      continue;
    }
    const int slot0 = j0 % page_size;
    const T* kbase = cache + kv_offset(page, 0, hk, slot0, n_kv_head, page_size, head_dim);
    const T* vbase = cache + kv_offset(page, 1, hk, slot0, n_kv_head, page_size, head_dim);
    const int j = j0 + key_in_unit;
    const bool valid = j >= k_begin && j < k_end;
    float dot = 0.0f;
    if (valid) {
      const T* kr = kbase + (size_t)key_in_unit * head_dim;
      for (int c = half; c < n_pieces; c += 2) dot += Vec16<T>::dot(kr + c * VN, qs + c * VN);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float s = valid ? dot * scale : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.0f;
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    // every key's p sits in two lanes: halve the warp sum
    l = l * corr + 0.5f * warp_sum(p);
#pragma unroll
    for (int i = 0; i < 2 * DEC_MAX_PAIRS; ++i) o[i] *= corr;
    const int jj_lo = max(k_begin - j0, 0), jj_hi = min(k_end - j0, 16);
    for (int jj = jj_lo; jj < jj_hi; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj * 2);
      const T* vr = vbase + (size_t)jj * head_dim;
#pragma unroll
      for (int i = 0; i < DEC_MAX_PAIRS; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < head_dim) {
          const float2 v = load2(vr + d);
          o[2 * i] = fmaf(pj, v.x, o[2 * i]);
          o[2 * i + 1] = fmaf(pj, v.y, o[2 * i + 1]);
        }
      }
    }
    m = m_new;
  }
  // merge the warps of the block, in warp order
  if (lane == 0) {
    wm[warp] = m;
    wl[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < DEC_MAX_PAIRS; ++i) {
    const int d = 2 * lane + 64 * i;
    if (d < head_dim) {
      wo[warp * head_dim + d] = o[2 * i];
      wo[warp * head_dim + d + 1] = o[2 * i + 1];
    }
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w]);
  float L = 0.0f;
  float f[DEC_WARPS];
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    f[w] = (wm[w] == -INFINITY) ? 0.0f : expf(wm[w] - M);
    L += wl[w] * f[w];
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.0f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) acc += wo[w * head_dim + d] * f[w];
    if (n_splits == 1)
      out[(size_t)t * ldo + h * head_dim + d] = from_float<T>(acc / L);
    else
      part_o[pidx * head_dim + d] = acc;
  }
  if (n_splits > 1 && threadIdx.x == 0) {
    part_ml[2 * pidx] = M;
    part_ml[2 * pidx + 1] = L;
  }
}

template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       T* __restrict__ out, int ldo, const int* __restrict__ rows, int n_head,
                                       int head_dim, int n_splits) {
  const int h = blockIdx.x, r = blockIdx.y;
  const int t = rows ? rows[r] : r;
  const size_t base = ((size_t)r * n_head + h) * n_splits;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[2 * (base + s)]);
  float L = 0.0f;
  for (int s = 0; s < n_splits; ++s) {
    const float ls = part_ml[2 * (base + s) + 1];
    if (ls > 0.0f) L += ls * expf(part_ml[2 * (base + s)] - M);
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
      const float ls = part_ml[2 * (base + s) + 1];
      if (ls > 0.0f) acc += part_o[(base + s) * head_dim + d] * expf(part_ml[2 * (base + s)] - M);
    }
    out[(size_t)t * ldo + h * head_dim + d] = from_float<T>(acc / L);
  }
}

template <typename T>
static int launch_decode(const void* q, int ldq, const void* cache, float* part_o, float* part_ml, void* out,
                         int ldo, const int* block_table, int max_blocks, const int* rows, const int* row_entry,
                         const int* positions, int n_rows, int n_head, int n_kv_head, int head_dim,
                         int page_size, int n_pages, float scale, int window, int chunk, int n_splits,
                         int* status, cudaStream_t stream) {
  dim3 grid(n_splits, n_head, n_rows);
  const size_t smem = (size_t)(head_dim + DEC_WARPS * head_dim + 2 * DEC_WARPS) * sizeof(float);
  attention_decode_kernel<T><<<grid, DEC_WARPS * 32, smem, stream>>>(
      (const T*)q, ldq, (const T*)cache, part_o, part_ml, (T*)out, ldo, block_table, max_blocks, rows, row_entry,
      positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, chunk, n_splits, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (n_splits > 1) {
    dim3 mgrid(n_head, n_rows);
    attention_merge_kernel<T><<<mgrid, 64, 0, stream>>>(part_o, part_ml, (T*)out, ldo, rows, n_head, head_dim,
                                                         n_splits);
  }
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

// Floats of scratch that nib_attention_decode needs for its partial results.
extern "C" long long nib_attention_decode_scratch(int n_rows, int n_head, int head_dim, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)n_rows * n_head * n_splits * (head_dim + 2);
}

// rows: indices of the step's rows to process (nullptr: rows 0..n_rows-1).  Keys are split into
// chunks of `chunk` positions (a multiple of 16); n_splits = ceil(longest key range / chunk).
// scratch holds nib_attention_decode_scratch(...) floats.
extern "C" int nib_attention_decode(int dtype, const void* q, int ldq, const void* cache, float* scratch,
                                    void* out, int ldo, const int* block_table, int max_blocks, const int* rows,
                                    const int* row_entry, const int* positions, int n_rows, int n_head,
                                    int n_kv_head, int head_dim, int page_size, int n_pages, float scale,
                                    int window, int chunk, int n_splits, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (head_dim <= 0 || head_dim > 64 * DEC_MAX_PAIRS || (head_dim & 7)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (page_size % 16 != 0 || chunk <= 0 || chunk % 16 != 0 || n_splits <= 0) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0) return NIB_ERR_BAD_ARGUMENT;
  if (n_rows > 65535 || n_head > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_splits > 1 && scratch == nullptr) return NIB_ERR_BAD_ARGUMENT;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)n_rows * n_head * n_splits * head_dim : nullptr;
  if (dtype == DT_F32)
    return launch_decode<float>(q, ldq, cache, part_o, part_ml, out, ldo, block_table, max_blocks, rows, row_entry,
                                positions, n_rows, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window,
                                chunk, n_splits, status, stream);
  if (dtype == DT_BF16)
    return launch_decode<bf16>(q, ldq, cache, part_o, part_ml, out, ldo, block_table, max_blocks, rows, row_entry,
                               positions, n_rows, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window,
                               chunk, n_splits, status, stream);
  return NIB_ERR_BAD_ARGUMENT;
}
