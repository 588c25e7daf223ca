// Attention for single decoded tokens: split-KV "flash decoding" over the block tables.
//
// One block handles one (row, head, split of the keys): it streams its share of the paged keys
// and values once, keeps an online softmax (running maximum m, sum l, unnormalised output o) and
// writes the partial (m, l, o); the block of a (row, head) that finishes last merges its splits in
// split order:  M = max m_s;  L = sum l_s e^(m_s - M);  out = sum o_s e^(m_s - M) / L.
// This is the reference's b_attn_split / b_attn_merge pair
// (crates/metal/src/shaders/batch.metal:349-424) with the split size chosen by the host so that
// a small batch still fills the GPU.  Scores are (q . k) * scale for the keys lo..pos, in 32-bit
// (crates/core/src/kernels/reference.rs:109-142).
//
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int DEC_WARPS = 4;
constexpr int DEC_MAX_HD = 128;

template <typename T> struct Piece;  // one 16-byte piece of a key or value row
template <> struct Piece<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void unpack(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
};
template <> struct Piece<bf16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void unpack(float* f) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};

// partial layout: o [row][head][split][head_dim], ml [row][head][split][2]
//
// Inside a warp, lanes 2s and 2s+1 own key slot s of every 16-key unit: they split the 16-byte
// pieces of the key row (and of the value row) between them, so a unit is 32 lanes x several
// independent 16-byte loads.  Each lane pair keeps an online softmax of its own over its keys
// (no exchange between lanes inside the loop but the one that completes the dot product); the
// sixteen pairs, then the four warps, are merged once at the end, in a fixed order.
// Units of sixteen keys whose loads a warp keeps in flight together (fewer when a lane holds many pieces).
#ifndef NIB_DEC_UNITS
#define NIB_DEC_UNITS 1
#endif
#define NIB_DEC_UNITS_FOR(pieces) ((pieces) <= 4 ? NIB_DEC_UNITS : 1)

template <typename T, int HD_MAX>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache, float* __restrict__ part_o,
                        float* __restrict__ part_ml, T* __restrict__ out, int ldo,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ rows,
                        const int* __restrict__ row_entry, const int* __restrict__ positions, int n_head,
                        int n_kv_head, int head_dim, int page_size, int n_pages, float scale, int window,
                        int chunk, int n_splits, int* __restrict__ counters, int* __restrict__ status) {
  constexpr int VN = Piece<T>::N;
  constexpr int MAXP = HD_MAX / VN / 2;   // pieces per lane
  pdl_trigger();
  extern __shared__ float smem[];
  float* qs = smem;                                  // head_dim
  float* wo = smem + head_dim;                       // DEC_WARPS * head_dim
  float* wm = wo + DEC_WARPS * head_dim;             // DEC_WARPS
  float* wl = wm + DEC_WARPS;                        // DEC_WARPS
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  // The step's tables were written before the step began and the cache below this row's position
  // belongs to earlier steps: both may be read before the kernel ahead (which writes this row's own
  // key and value, and the queries) has finished.
  const int t = rows ? rows[r] : r;
  const int pos = positions[t];
  const int* table = block_table + (size_t)row_entry[t] * max_blocks;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);  // exclusive
  const int hk = h / (n_head / n_kv_head);
  const size_t pidx = ((size_t)r * n_head + h) * n_splits + split;
  __shared__ int is_last_sh;
  const bool empty = k_begin >= k_end;  // nothing in this split: the merge skips l == 0

  const int n_pieces = head_dim / VN;  // 16-byte pieces per row
  const int slot_in_unit = lane >> 1, half = lane & 1;
  // units of 16 consecutive keys that lie in one page (page_size is a multiple of 16)
  const int first_unit = empty ? 0 : k_begin / 16, last_unit = empty ? -1 : (k_end - 1) / 16;
  // This warp's units are first_unit + warp + i * DEC_WARPS; it works on them in groups of UNITS
  // whose loads are all in flight together.
  constexpr int UNITS = NIB_DEC_UNITS_FOR(MAXP);
  const int n_mine = (first_unit + warp <= last_unit) ? (last_unit - first_unit - warp) / DEC_WARPS + 1 : 0;
  Piece<T> kp[UNITS][MAXP], vp[UNITS][MAXP];
  bool act[UNITS];
  // asks for this lane pair's key and value pieces of the group that starts at the warp's unit i0
  auto fetch = [&](int i0) {
#pragma unroll
    for (int uu = 0; uu < UNITS; ++uu) {
      act[uu] = false;
      if (i0 + uu >= n_mine) continue;
      const int j0 = (first_unit + warp + (i0 + uu) * DEC_WARPS) * 16;
      const int page = table[j0 / page_size];
      if (page < 0 || page >= n_pages) {
        if (lane == 0) *status = NIB_STATUS_BAD_PAGE;
        continue;
      }
      const int j = j0 + slot_in_unit;
      if (j < k_begin || j >= k_end) continue;
      act[uu] = true;
      const int slot = j % page_size;
      const T* kr = cache + kv_offset(page, 0, hk, slot, n_kv_head, page_size, head_dim);
      const T* vr = cache + kv_offset(page, 1, hk, slot, n_kv_head, page_size, head_dim);
#pragma unroll
      for (int i = 0; i < MAXP; ++i) {
        const int c = half + 2 * i;
        if (c < n_pieces) {
          kp[uu][i].load(kr + c * VN);
          vp[uu][i].load(vr + c * VN);
        }
      }
    }
  };
  // none of the first group's keys is the one that the kernel ahead writes
  const int first_group_last = first_unit + warp + (min(UNITS, n_mine) - 1) * DEC_WARPS;
  const bool early = n_mine > 0 && first_group_last * 16 + 15 < pos;
  if (early) fetch(0);
  pdl_wait();

  if (empty) {
    if (threadIdx.x == 0) {
      part_ml[2 * pidx] = -INFINITY;
      part_ml[2 * pidx + 1] = 0.0f;
    }
  } else {
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = to_float(q[(size_t)t * ldq + h * head_dim + d]);
  __syncthreads();

  float o[MAXP * VN];
#pragma unroll
  for (int i = 0; i < MAXP * VN; ++i) o[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;

  for (int i0 = 0; i0 < n_mine; i0 += UNITS) {
    if (i0 > 0 || !early) fetch(i0);
#pragma unroll
    for (int uu = 0; uu < UNITS; ++uu) {
      if (!act[uu]) continue;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < MAXP; ++i) {
        const int c = half + 2 * i;
        if (c < n_pieces) {
          float f[VN];
          kp[uu][i].unpack(f);
#pragma unroll
          for (int e = 0; e < VN; ++e) dot = fmaf(f[e], qs[c * VN + e], dot);
        }
      }
      // both lanes of the pair are here together (whether a pair has a key depends on the pair only)
      dot += __shfl_xor_sync(0x3u << (lane & ~1), dot, 1);
      const float s = dot * scale;
      const float m_new = fmaxf(m, s);
      const float p = expf(s - m_new);
      const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
      l = l * corr + p;
      m = m_new;
#pragma unroll
      for (int i = 0; i < MAXP; ++i) {
        const int c = half + 2 * i;
        if (c < n_pieces) {
          float f[VN];
          vp[uu][i].unpack(f);
#pragma unroll
          for (int e = 0; e < VN; ++e) o[i * VN + e] = fmaf(p, f[e], o[i * VN + e] * corr);
        }
      }
    }
  }
  __syncwarp();
  // ---- merge the sixteen lane pairs of the warp
  const float mw = warp_max(m);
  const float f_lane = (m == -INFINITY) ? 0.0f : expf(m - mw);
  float lw = (half == 0) ? l * f_lane : 0.0f;
  lw = warp_sum(lw);
#pragma unroll
  for (int i = 0; i < MAXP * VN; ++i) {
    float v = o[i] * f_lane;
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    o[i] = v;
  }
  if (lane == 0) {
    wm[warp] = mw;
    wl[warp] = lw;
  }
  if (slot_in_unit == 0) {
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int c = half + 2 * i;
      if (c < n_pieces) {
#pragma unroll
        for (int e = 0; e < VN; ++e) wo[warp * head_dim + c * VN + e] = o[i * VN + e];
      }
    }
  }
  __syncthreads();
  // ---- merge the warps of the block, in warp order
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
  }  // !empty
  if (n_splits == 1) return;
  // ---- the block that finishes last merges the splits of its (row, head), in split order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(&counters[r * n_head + h], 1);
    is_last_sh = arrived == n_splits - 1;
    if (is_last_sh) counters[r * n_head + h] = 0;  // zero again for the next launch
  }
  __syncthreads();
  if (!is_last_sh) return;
  __threadfence();
  const size_t base = ((size_t)r * n_head + h) * n_splits;
  float Mx = -INFINITY;
  for (int sp = 0; sp < n_splits; ++sp) Mx = fmaxf(Mx, part_ml[2 * (base + sp)]);
  float Lx = 0.0f;
  for (int sp = 0; sp < n_splits; ++sp) {
    const float ls = part_ml[2 * (base + sp) + 1];
    if (ls > 0.0f) Lx += ls * expf(part_ml[2 * (base + sp)] - Mx);
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float ls = part_ml[2 * (base + sp) + 1];
      if (ls > 0.0f) acc += part_o[(base + sp) * head_dim + d] * expf(part_ml[2 * (base + sp)] - Mx);
    }
    out[(size_t)t * ldo + h * head_dim + d] = from_float<T>(acc / Lx);
  }
}

template <typename T>
static int launch_decode(const void* q, int ldq, const void* cache, float* part_o, float* part_ml, void* out,
                         int ldo, const int* block_table, int max_blocks, const int* rows, const int* row_entry,
                         const int* positions, int n_rows, int n_head, int n_kv_head, int head_dim,
                         int page_size, int n_pages, float scale, int window, int chunk, int n_splits,
                         int* counters, int* status, cudaStream_t stream) {
  dim3 grid(n_splits, n_head, n_rows);
  const size_t smem = (size_t)(head_dim + DEC_WARPS * head_dim + 2 * DEC_WARPS) * sizeof(float);
  if (head_dim <= 64)
    launch_pdl(attention_decode_kernel<T, 64>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, 
        (const T*)q, ldq, (const T*)cache, part_o, part_ml, (T*)out, ldo, block_table, max_blocks, rows, row_entry,
        positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, chunk, n_splits, counters, status);
  else
    launch_pdl(attention_decode_kernel<T, DEC_MAX_HD>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, 
        (const T*)q, ldq, (const T*)cache, part_o, part_ml, (T*)out, ldo, block_table, max_blocks, rows, row_entry,
        positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, chunk, n_splits, counters, status);
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
// scratch holds nib_attention_decode_scratch(...) floats; counters holds n_rows * n_head ints that are
// zero before the first call (the kernel leaves them zero).
extern "C" int nib_attention_decode(int dtype, const void* q, int ldq, const void* cache, float* scratch,
                                    void* out, int ldo, const int* block_table, int max_blocks, const int* rows,
                                    const int* row_entry, const int* positions, int n_rows, int n_head,
                                    int n_kv_head, int head_dim, int page_size, int n_pages, float scale,
                                    int window, int chunk, int n_splits, int* counters, int* status,
                                    cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (head_dim <= 0 || head_dim > DEC_MAX_HD || (head_dim & 7)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (page_size % 16 != 0 || chunk <= 0 || chunk % 16 != 0 || n_splits <= 0) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0) return NIB_ERR_BAD_ARGUMENT;
  if (n_rows > 65535 || n_head > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_splits > 1 && (scratch == nullptr || counters == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)n_rows * n_head * n_splits * head_dim : nullptr;
  if (dtype == DT_F32)
    return launch_decode<float>(q, ldq, cache, part_o, part_ml, out, ldo, block_table, max_blocks, rows, row_entry,
                                positions, n_rows, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window,
                                chunk, n_splits, counters, status, stream);
  if (dtype == DT_BF16)
    return launch_decode<bf16>(q, ldq, cache, part_o, part_ml, out, ldo, block_table, max_blocks, rows, row_entry,
                               positions, n_rows, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window,
                               chunk, n_splits, counters, status, stream);
  return NIB_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and described in attention_decode_static.h).
#include "attention_decode_static.h"

// Partial results first, then the arrival counters (as ints), in one array.
static __device__ __align__(256) float g_static_scratch[NIB_STATIC_SCRATCH_FLOATS + NIB_STATIC_COUNTERS];

// In host code the array's name is only a handle; its device address differs per GPU and is looked
// up once per device, with that device current.
static float* static_scratch_on_current_device(int* err) {
  constexpr int MAX_DEVICES = 64;
  static float* addr[MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    *err = e != cudaSuccess ? (int)e : NIB_ERR_BAD_ARGUMENT;
    return nullptr;
  }
  if (addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess) {
      *err = (int)e;
      return nullptr;
    }
    addr[dev] = p;
  }
  *err = 0;
  return addr[dev];
}

extern "C" void nib_attention_decode_static_limits(long long* max_floats, long long* max_counters) {
  if (max_floats) *max_floats = NIB_STATIC_SCRATCH_FLOATS;
  if (max_counters) *max_counters = NIB_STATIC_COUNTERS;
}

extern "C" int nib_attention_decode_static(int dtype, const void* q, int ldq, const void* cache, void* out,
                                           int ldo, const int* block_table, int max_blocks, const int* rows,
                                           const int* row_entry, const int* positions, int n_rows, int n_head,
                                           int n_kv_head, int head_dim, int page_size, int n_pages, float scale,
                                           int window, int chunk, int n_splits, int* status,
                                           cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_head <= 0 || n_splits <= 0 || head_dim <= 0) return NIB_ERR_BAD_ARGUMENT;
  const long long need_floats = nib_attention_decode_scratch(n_rows, n_head, head_dim, n_splits);
  const long long need_counters = (long long)n_rows * n_head;
  if (need_floats > NIB_STATIC_SCRATCH_FLOATS || need_counters > NIB_STATIC_COUNTERS)
    return NIB_ERR_STATIC_SCRATCH_TOO_SMALL;
  int err = 0;
  float* scratch = static_scratch_on_current_device(&err);
  if (scratch == nullptr) return err;
  int* counters = reinterpret_cast<int*>(scratch + NIB_STATIC_SCRATCH_FLOATS);
  // the counters are what must start at zero; an earlier call that was cut short may have left them otherwise
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)need_counters * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  return nib_attention_decode(dtype, q, ldq, cache, scratch, out, ldo, block_table, max_blocks, rows, row_entry,
                              positions, n_rows, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window,
                              chunk, n_splits, counters, status, stream);
}
