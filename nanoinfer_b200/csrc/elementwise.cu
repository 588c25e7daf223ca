// Embedding (+ learned positions), LayerNorm (with an optional row gather) and the
// append of new keys and values to the paged cache.
//
// Formulas: x[t] = wte[tok_t] + wpe[pos_t] (reference: crates/core/src/kernels/reference.rs:86-94);
// LayerNorm two-pass with biased variance, rstd = 1/sqrt(var + eps) (reference.rs:42-51);
// K/V rows of the fused qkv buffer copied to the cache slot of their position
// (crates/core/src/stages/kv_cache.rs:44-57, crates/metal/src/shaders/batch.metal:329-344).
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace nib {

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                             const T* __restrict__ table, const T* __restrict__ pos_table,
                             const int* feedback, float* out, int C) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0) tok = feedback[-tok - 1];   // the token that the step before sampled for slot -tok - 1
  const T* te = table + (size_t)tok * C;
  float* o = out + (size_t)t * C;
  if (pos_table != nullptr) {
    const T* pe = pos_table + (size_t)positions[t] * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = to_float(te[c]) + to_float(pe[c]);
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = to_float(te[c]);
  }
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

// ------------------------------------------------------------------ layernorm
// One block per output row.  The row is staged in shared memory as 32-bit floats,
// so the mean and the variance are two true passes over the same values.
template <typename OutT>
__global__ void layernorm_kernel(const float* x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 OutT* out, int C, float eps) {
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

// One warp per row, the row in registers (NV float4 per lane: C <= 128 * NV), eight rows a block: no
// shared memory and no block-wide barrier.  Same two true passes as above.
template <typename OutT, int NV>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ gamma,
                      const float* __restrict__ beta, OutT* out, int n_rows, int C, float eps) {
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  pdl_wait();
  if (r >= n_rows) return;
  const float* src = x + (size_t)(rows ? rows[r] : r) * C;
  float4 v[NV];
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int k = (j * 32 + lane) * 4;
    v[j] = k < C ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = warp_sum(s) / (float)C;
  float q = 0.0f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if ((j * 32 + lane) * 4 < C) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)C + eps);
  OutT* o = out + (size_t)r * C;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int k = (j * 32 + lane) * 4;
    if (k < C) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + k), b = *reinterpret_cast<const float4*>(beta + k);
      store4(o + k, (v[j].x - mean) * rstd * g.x + b.x, (v[j].y - mean) * rstd * g.y + b.y,
             (v[j].z - mean) * rstd * g.z + b.z, (v[j].w - mean) * rstd * g.w + b.w);
    }
  }
}

// ------------------------------------------------------------------ kv append
// src is the fused projection output [T, ld]; keys start at column k_off, values at v_off.
template <typename T>
__global__ void kv_append_kernel(const T* src, int ld, int k_off, int v_off,
                                 T* cache, const int* __restrict__ block_table,
                                 int max_blocks, const int* __restrict__ row_entry,
                                 const int* __restrict__ positions, int n_kv_head, int head_dim,
                                 int page_size, int n_pages, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int entry = row_entry[t];
  if (entry < 0) return;   // a row of no request (padding): nothing to keep
  const int pos = positions[t];
  const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
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

// The same in 16-byte pieces, one thread a piece, several rows a block (head_dim, ld and the offsets
// are multiples of the piece).
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_pieces_kernel(const T* src, int ld, int k_off, int v_off, T* cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_entry,
                        const int* __restrict__ positions, int n_rows, int n_kv_head, int head_dim, int page_size,
                        int n_pages, int* status) {
  constexpr int VN = 16 / sizeof(T);
  pdl_trigger();
  const int per_head = head_dim / VN, per_row = 2 * n_kv_head * per_head;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int t = (int)(idx / per_row), piece = (int)(idx - (long long)t * per_row);
  if (t >= n_rows) return;   // (exiting counts as having waited)
  const int entry = row_entry[t];
  if (entry < 0) return;     // a row of no request (padding): nothing to keep
  const int pos = positions[t];
  const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
  pdl_wait();
  if (page < 0 || page >= n_pages) {
    *status = NIB_STATUS_BAD_PAGE;
    return;
  }
  const int kv = piece / (n_kv_head * per_head), rem = piece - kv * n_kv_head * per_head;
  const int h = rem / per_head, d = (rem - h * per_head) * VN;
  const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)t * ld + (kv ? v_off : k_off) + h * head_dim + d);
  *reinterpret_cast<uint4*>(cache + kv_offset(page, kv, h, pos % page_size, n_kv_head, page_size, head_dim) + d) = v;
}

}  // namespace nib

using namespace nib;

extern "C" int nib_embed(int dtype, const int* tokens, const int* positions, const void* table,
                         const void* pos_table, const int* feedback, float* out, int T, int C,
                         cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = C >= 256 ? 256 : 128;
  if (dtype == DT_F32)
    launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, tokens, positions, (const float*)table,
                                                   (const float*)pos_table, feedback, out, C);
  else if (dtype == DT_BF16)
    launch_pdl(embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, tokens, positions, (const bf16*)table,
                                                  (const bf16*)pos_table, feedback, out, C);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

template <typename OutT>
static int launch_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, OutT* out,
                            int n_rows, int C, float eps, cudaStream_t stream) {
  const bool vec = (C & 3) == 0 && C <= 2048 && (((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0 &&
                   ((uintptr_t)out & (4 * sizeof(OutT) - 1)) == 0;
  if (vec) {   // whatever the number of rows: a row's result must not depend on it
    const dim3 grid((n_rows + 7) / 8);
    if (C <= 1024)
      launch_pdl(layernorm_rows_kernel<OutT, 8>, grid, dim3(256), 0, stream, x, rows, gamma, beta, out, n_rows, C, eps);
    else
      launch_pdl(layernorm_rows_kernel<OutT, 16>, grid, dim3(256), 0, stream, x, rows, gamma, beta, out, n_rows, C, eps);
    NIB_LAUNCH_CHECK();
  }
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const int threads = C >= 1024 ? 512 : (C >= 256 ? 256 : 128);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(layernorm_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(layernorm_kernel<OutT>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, out, C, eps);
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_layernorm(int out_dtype, const float* x, const int* rows, const float* gamma,
                             const float* beta, void* out, int n_rows, int C, float eps,
                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (out_dtype == DT_F32) return launch_layernorm<float>(x, rows, gamma, beta, (float*)out, n_rows, C, eps, stream);
  if (out_dtype == DT_BF16) return launch_layernorm<bf16>(x, rows, gamma, beta, (bf16*)out, n_rows, C, eps, stream);
  return NIB_ERR_BAD_ARGUMENT;
}

template <typename T>
static int launch_kv_append(const T* src, int ld, int k_off, int v_off, T* cache, const int* block_table,
                            int max_blocks, const int* row_entry, const int* positions, int n_rows, int n_kv_head,
                            int head_dim, int page_size, int n_pages, int* status, cudaStream_t stream) {
  constexpr int VN = 16 / sizeof(T);
  const bool pieces = head_dim % VN == 0 && ld % VN == 0 && k_off % VN == 0 && v_off % VN == 0 &&
                      (((uintptr_t)src | (uintptr_t)cache) & 15) == 0;
  if (pieces) {
    const long long total = (long long)n_rows * 2 * n_kv_head * (head_dim / VN);
    launch_pdl(kv_append_pieces_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, src, ld, k_off,
               v_off, cache, block_table, max_blocks, row_entry, positions, n_rows, n_kv_head, head_dim, page_size,
               n_pages, status);
  } else {
    launch_pdl(kv_append_kernel<T>, dim3(n_rows), dim3(128), 0, stream, src, ld, k_off, v_off, cache, block_table,
               max_blocks, row_entry, positions, n_kv_head, head_dim, page_size, n_pages, status);
  }
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_kv_append(int dtype, const void* src, int ld, int k_off, int v_off, void* cache,
                             const int* block_table, int max_blocks, const int* row_entry,
                             const int* positions, int T, int n_kv_head, int head_dim,
                             int page_size, int n_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == DT_F32)
    return launch_kv_append<float>((const float*)src, ld, k_off, v_off, (float*)cache, block_table, max_blocks,
                                   row_entry, positions, T, n_kv_head, head_dim, page_size, n_pages, status, stream);
  if (dtype == DT_BF16)
    return launch_kv_append<bf16>((const bf16*)src, ld, k_off, v_off, (bf16*)cache, block_table, max_blocks,
                                  row_entry, positions, T, n_kv_head, head_dim, page_size, n_pages, status, stream);
  return NIB_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// Loading: a checkpoint tensor's rows, as the file stores them (32-bit or 16-bit floats), into the
// engine's tensor: converted, and transposed where the file stores a matrix [in, out]
// (crates/core/src/weights.rs:48-57 transposes on the host; here the bytes go to the device as they
// lie in the file and this kernel puts them in place).
namespace nib {

enum : int { SRC_F32 = 0, SRC_BF16 = 1, SRC_F16 = 2 };

__device__ __forceinline__ float load_as_float(const void* src, int src_dt, size_t i) {
  if (src_dt == SRC_F32) return reinterpret_cast<const float*>(src)[i];
  if (src_dt == SRC_BF16) return __bfloat162float(reinterpret_cast<const bf16*>(src)[i]);
  return __half2float(reinterpret_cast<const __half*>(src)[i]);
}

// src: [rows, cols] as stored.  dst (row stride ld): element (r, c) goes to dst[(r0 + r) * ld + c], or
// with `transpose` to dst[c * ld + r0 + r]; tiles of 32 x 32 pass through shared memory so that both
// sides are read and written along their rows.
template <typename D>
__global__ void convert_kernel(const void* __restrict__ src, int src_dt, int rows, int cols, D* __restrict__ dst,
                               long long ld, long long r0, int transpose) {
  __shared__ float tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;   // first column, first row of the tile
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, c = bx + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < cols) ? load_as_float(src, src_dt, (size_t)r * cols + c) : 0.0f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    if (!transpose) {
      const int r = by + j, c = bx + threadIdx.x;
      if (r < rows && c < cols) dst[(size_t)(r0 + r) * ld + c] = from_float<D>(tile[j][threadIdx.x]);
    } else {
      const int c = bx + j, r = by + threadIdx.x;         // the tile read the other way round
      if (r < rows && c < cols) dst[(size_t)c * ld + r0 + r] = from_float<D>(tile[threadIdx.x][j]);
    }
  }
}

}  // namespace nib

extern "C" int nib_convert(int src_dtype, const void* src, int rows, int cols, int dst_dtype, void* dst,
                           long long ld, long long r0, int transpose, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (src_dtype < 0 || src_dtype > 2) return NIB_ERR_BAD_ARGUMENT;
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dst_dtype == DT_F32)
    convert_kernel<float><<<grid, block, 0, stream>>>(src, src_dtype, rows, cols, (float*)dst, ld, r0, transpose);
  else if (dst_dtype == DT_BF16)
    convert_kernel<bf16><<<grid, block, 0, stream>>>(src, src_dtype, rows, cols, (bf16*)dst, ld, r0, transpose);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
