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
  __device__ __forceinline__ void load(const void* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void unpack(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
};
template <> struct Piece<bf16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void load(const void* p) { raw = *reinterpret_cast<const uint4*>(p); }
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

// 2^x.  The bfloat16 kernel takes the hardware's approximation (relative error about 2^-22, far below
// the rounding of the values it multiplies; 2^-inf = 0); the 32-bit kernel takes the accurate library
// function, as the general attention kernel that serves its prompt portions does, so that no
// approximate instruction stands anywhere in the true 32-bit path.
template <typename T> __device__ __forceinline__ float pow2(float x);
template <> __device__ __forceinline__ float pow2<bf16>(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <> __device__ __forceinline__ float pow2<float>(float x) { return exp2f(x); }

// partial layout: o [row][head][split][head_dim], ml [row][head][split][2]
//
// A (page, K|V, head) of the cache is a contiguous run of rows, so a warp reads it as a plain
// stream: LPR lanes stand side by side on one key row (a 16-byte piece each; LPR is the power of
// two that covers the row), the 32 / LPR lane groups of the warp on consecutive rows, and one load
// instruction of the warp covers whole 128-byte lines.  (Lanes spread over many rows with a piece
// of each ask for a 32-byte sector per line and instruction, which halves what the memory system
// delivers.)  A lane keeps the score products of its piece, the group completes them with
// shuffles; every group runs an online softmax of its own over its keys, BATCH keys at a time, and
// keeps the output for its lanes' pieces.  The groups, then the warps, are merged once at the end,
// in a fixed order.
// (q, cache and out carry no __restrict__: the kernel ahead writes them; see pdl_wait in common.cuh)
template <typename T, int LPR>
__global__ void __launch_bounds__(DEC_WARPS * 32, 6)   // six blocks an SM: what the host's choice of splits counts on
attention_decode_kernel(const T* q, int ldq, const T* cache, float* part_o,
                        float* part_ml, T* out, int ldo,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ rows,
                        const int* __restrict__ row_entry, const int* __restrict__ positions, int n_head,
                        int n_kv_head, int head_dim, int page_size, int n_pages, float scale, int window,
                        int chunk, int n_splits, int* counters, int* status,
                        int cluster_merge) {
  constexpr int VN = Piece<T>::N;
  constexpr int BATCH = LPR / 2 < 4 ? LPR / 2 : 4;   // keys per lane group and batch
  constexpr int GROUPS = 32 / LPR;                   // lane groups of a warp: rows per load instruction
  constexpr int BK = BATCH * GROUPS;                 // keys per batch of a warp: 16, 8 or 4
  constexpr int ALL_GROUPS = DEC_WARPS * GROUPS;
  pdl_trigger();
  extern __shared__ __align__(16) float smem[];
  float* go = smem;                                  // ALL_GROUPS * head_dim
  float* gm = go + ALL_GROUPS * head_dim;            // ALL_GROUPS
  float* gl = gm + ALL_GROUPS;                       // ALL_GROUPS
  // When the splits of a (row, head) are the blocks of one cluster, they hand their results to the
  // first of them through distributed shared memory instead of through global scratch and a counter.
  float* xo = gl + ALL_GROUPS;                       // n_splits * head_dim (used in block 0 of the cluster)
  float* xml = xo + n_splits * head_dim;             // n_splits * 2
  if (cluster_merge) cluster_arrive();               // met below, before the first store into another block
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

  const int group = lane / LPR, c = lane % LPR;
  const bool has_piece = c * VN < head_dim;
  // batches of BK consecutive keys (BK divides 16, so a batch lies in one page); this warp's batches
  // are first_batch + warp + i * DEC_WARPS
  const int first_batch = empty ? 0 : k_begin / BK, last_batch = empty ? -1 : (k_end - 1) / BK;
  const int n_mine = (first_batch + warp <= last_batch) ? (last_batch - first_batch - warp) / DEC_WARPS + 1 : 0;
  Piece<T> kp[BATCH], vp[BATCH];
  uint32_t live = 0;   // bit i: key i of the batch in kp/vp is one of this split's
  // where this lane's piece of a row lies: ((page * 2 + K|V) * n_kv_head + head) * page_size + slot) * head_dim + piece
  const size_t kv_stride = (size_t)n_kv_head * page_size * head_dim;
  const T* lane_base = cache + ((size_t)hk * page_size + group) * head_dim + c * VN;
  // asks for this lane's pieces of the warp's batch i
  auto fetch = [&](int i) {
    const int j0 = (first_batch + warp + i * DEC_WARPS) * BK;
    const int page = table[page_size == 16 ? (j0 >> 4) : j0 / page_size];
    live = 0;
    if (page < 0 || page >= n_pages) {
      if (lane == 0) *status = NIB_STATUS_BAD_PAGE;
      return;
    }
    const int slot0 = page_size == 16 ? (j0 & 15) : j0 % page_size;
    const T* kr = lane_base + (size_t)page * 2 * kv_stride + (size_t)slot0 * head_dim;
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int j = j0 + b * GROUPS + group;
      if (j >= k_begin && j < k_end) {
        live |= 1u << b;
        if (has_piece) {
          kp[b].load(kr + b * GROUPS * head_dim);
          vp[b].load(kr + b * GROUPS * head_dim + kv_stride);
        }
      }
    }
  };
  // none of the first batch's keys is the one that the kernel ahead writes
  const bool early = n_mine > 0 && (first_batch + warp) * BK + BK - 1 < pos;
  if (early) fetch(0);
  pdl_wait();
  if (cluster_merge) cluster_wait();   // every block of the cluster runs by now

  if (empty) {
    if (threadIdx.x == 0) {
      if (cluster_merge) {
        store_to_rank(xml + 2 * split, 0, -INFINITY);
        store_to_rank(xml + 2 * split + 1, 0, 0.0f);
      } else {
        part_ml[2 * pidx] = -INFINITY;
        part_ml[2 * pidx + 1] = 0.0f;
      }
    }
  } else {
  float qf[VN];   // this lane's piece of the query
  {
    Piece<T> qp;
    if (has_piece) {
      qp.load(q + (size_t)t * ldq + h * head_dim + c * VN);
      qp.unpack(qf);
    } else {
#pragma unroll
      for (int e = 0; e < VN; ++e) qf[e] = 0.0f;
    }
  }
  float o[VN];
#pragma unroll
  for (int e = 0; e < VN; ++e) o[e] = 0.0f;
  // scores are kept times log2(e), so that the exponentials are plain powers of two
  const float scale2 = scale * 1.4426950408889634f;
  float m = -INFINITY, l = 0.0f;

  for (int i = 0; i < n_mine; ++i) {
    if (i > 0 || !early) fetch(i);
    float sc[BATCH];
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      float dot = 0.0f;
      if (((live >> b) & 1u) && has_piece) {
        float f[VN];
        kp[b].unpack(f);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot = fmaf(f[e], qf[e], dot);
      }
#pragma unroll
      for (int d = 1; d < LPR; d <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);   // the group's lanes, in a fixed order
      sc[b] = ((live >> b) & 1u) ? dot * scale2 : -INFINITY;
    }
    float m_new = m;
#pragma unroll
    for (int b = 0; b < BATCH; ++b) m_new = fmaxf(m_new, sc[b]);
    if (m_new == -INFINITY) continue;   // the group has had no key yet
    const float corr = pow2<T>(m - m_new);  // (2^-inf = 0 for the first keys)
    m = m_new;
    l *= corr;
#pragma unroll
    for (int e = 0; e < VN; ++e) o[e] *= corr;
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const float p = pow2<T>(sc[b] - m);   // 0 for a key that is not there
      l += p;
      if (has_piece && ((live >> b) & 1u)) {
        float f[VN];
        vp[b].unpack(f);
#pragma unroll
        for (int e = 0; e < VN; ++e) o[e] = fmaf(p, f[e], o[e]);
      }
    }
  }
  // ---- the lane groups' results meet in shared memory and are merged in group order
  const int g = warp * GROUPS + group;
  if (c == 0) {
    gm[g] = m;
    gl[g] = l;
  }
  if (has_piece) {
#pragma unroll
    for (int e = 0; e < VN; e += 4)
      *reinterpret_cast<float4*>(go + g * head_dim + c * VN + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < ALL_GROUPS; ++w) M = fmaxf(M, gm[w]);
  float L = 0.0f;
  for (int w = 0; w < ALL_GROUPS; ++w) L += (gm[w] == -INFINITY) ? 0.0f : gl[w] * pow2<T>(gm[w] - M);
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int w = 0; w < ALL_GROUPS; ++w) acc += (gm[w] == -INFINITY) ? 0.0f : go[w * head_dim + d] * pow2<T>(gm[w] - M);
    if (n_splits == 1)
      out[(size_t)t * ldo + h * head_dim + d] = from_float<T>(acc / L);
    else if (cluster_merge)
      store_to_rank(xo + split * head_dim + d, 0, acc);
    else
      part_o[pidx * head_dim + d] = acc;
  }
  if (n_splits > 1 && threadIdx.x == 0) {
    if (cluster_merge) {
      store_to_rank(xml + 2 * split, 0, M);
      store_to_rank(xml + 2 * split + 1, 0, L);
    } else {
      part_ml[2 * pidx] = M;      // (in the power-of-two scale)
      part_ml[2 * pidx + 1] = L;
    }
  }
  }  // !empty
  if (n_splits == 1) return;
  size_t base = ((size_t)r * n_head + h) * n_splits;
  if (cluster_merge) {
    // ---- the first block of the cluster merges the splits, in split order
    cluster_arrive();
    cluster_wait();
    if (split != 0) return;
    part_o = xo;
    part_ml = xml;
    base = 0;
  } else {
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
  }
  float Mx = -INFINITY;
  for (int sp = 0; sp < n_splits; ++sp) Mx = fmaxf(Mx, part_ml[2 * (base + sp)]);
  float Lx = 0.0f;
  for (int sp = 0; sp < n_splits; ++sp) {
    const float ls = part_ml[2 * (base + sp) + 1];
    if (ls > 0.0f) Lx += ls * pow2<T>(part_ml[2 * (base + sp)] - Mx);
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float ls = part_ml[2 * (base + sp) + 1];
      if (ls > 0.0f) acc += part_o[(base + sp) * head_dim + d] * pow2<T>(part_ml[2 * (base + sp)] - Mx);
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
  const int n_pieces = head_dim / Piece<T>::N;
  // two or four splits run as one cluster and merge through distributed shared memory (clusters of
  // eight measured slower than the merge through global scratch: they are harder to place)
  const int cluster = (n_splits == 2 || n_splits == 4) ? n_splits : 1;
#define NIB_DECODE_LAUNCH(LPR)                                                                                     \
  launch_pdl_cluster(attention_decode_kernel<T, LPR>, dim3(grid), dim3(DEC_WARPS * 32),                            \
             (size_t)(DEC_WARPS * (32 / LPR) * (head_dim + 2) + n_splits * (head_dim + 2)) * sizeof(float), stream, \
             cluster, (const T*)q, ldq, (const T*)cache, part_o, part_ml, (T*)out, ldo, block_table, max_blocks,   \
             rows, row_entry, positions, n_head, n_kv_head, head_dim, page_size, n_pages, scale, window, chunk,    \
             n_splits, counters, status, cluster > 1 ? 1 : 0)
  if (n_pieces <= 2) NIB_DECODE_LAUNCH(2);
  else if (n_pieces <= 4) NIB_DECODE_LAUNCH(4);
  else if (n_pieces <= 8) NIB_DECODE_LAUNCH(8);
  else if (n_pieces <= 16) NIB_DECODE_LAUNCH(16);
  else NIB_DECODE_LAUNCH(32);
#undef NIB_DECODE_LAUNCH
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
