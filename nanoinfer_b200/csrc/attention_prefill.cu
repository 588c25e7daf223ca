// Causal attention for prompt portions in bfloat16: a tiled flash kernel over the paged cache.
//
// One block takes 64 consecutive query rows of one request and one head; two warps share each 16
// rows, one for each half of a tile's 64 keys (a block's time is its longest chain of tiles, so the
// chain is made of half-size links), and their two softmax states are merged at the end.  Keys and
// values are gathered page by page into shared memory with cp.async (two buffers, the next tile
// loads while this one is computed); scores S = Q K^T and the weighted
// sum O += P V run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit accumulate); the
// softmax is online over tiles of 64 keys, in 32-bit, with the scale applied after the dot
// product and the causal bound as a loop bound plus a mask on the tiles that straddle it
// (crates/core/src/kernels/reference.rs:109-142; the tiling follows the reference's
// attn_prefill_flash, crates/metal/src/shaders/attn.metal:100-218, which reads a contiguous cache
// and fixes the head size at 64).  Several requests share a launch: the host lists the tiles as
// (entry, first row within the entry).
//
// The warp-level MMA keeps S and P in registers, which the softmax between the two products wants;
// the head size 64 of this architecture gives the 128-row tcgen05 shapes little to work on.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int PF_BM = 64;   // query rows per block
constexpr int PF_BN = 64;   // keys per tile
constexpr int PF_KSPLIT = 2;  // warps that share a row group, each with a part of a tile's keys
constexpr int PF_THREADS = 128 * PF_KSPLIT;
constexpr int PF_WN = PF_BN / PF_KSPLIT;   // keys per warp and tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware's approximation (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float pow2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const bf16* q, int ldq, const bf16* cache, bf16* out,
                         int ldo, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ tiles, const int* __restrict__ entry_start,
                         const int* __restrict__ entry_pos0, int n_head, int n_kv_head, int page_size, int n_pages,
                         float scale, int window, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  constexpr int LD = HD + 8;               // padded row: ldmatrix reads without bank conflicts
  constexpr int CHUNKS = HD / 8;           // 16-byte pieces per row
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);         // [PF_BM][LD]
  bf16* ks = qs + PF_BM * LD;                            // [2][PF_BN][LD]
  bf16* vs = ks + 2 * PF_BN * LD;                        // [2][PF_BN][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // (heads are the fast index of the grid: blocks start in the order of the tile list, longest first)
  const int e = tiles[2 * blockIdx.y], q_off = tiles[2 * blockIdx.y + 1];
  const int h = blockIdx.x, hk = h / (n_head / n_kv_head);
  const int row0 = entry_start[e] + q_off;               // first row of the tile in the step
  const int n_rows = min(PF_BM, entry_start[e + 1] - row0);
  const int pos_first = entry_pos0[e] + q_off;           // position of the tile's first row
  const int pos_last = pos_first + n_rows - 1;
  const int* table = block_table + (size_t)e * max_blocks;
  const int key_lo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int tile_first = key_lo / PF_BN, tile_last = pos_last / PF_BN;

  // ---- Q tile -> shared memory (rows past the request's end are zeros)
  for (int c = tid; c < PF_BM * CHUNKS; c += PF_THREADS) {
    const int r = c / CHUNKS, piece = c % CHUNKS;
    const bool valid = r < n_rows;
    const bf16* src = q + (size_t)(row0 + (valid ? r : 0)) * ldq + h * HD + piece * 8;
    cp_async16(qs + r * LD + piece * 8, src, valid);
  }
  // a row's place in the cache: (((page * 2 + K|V) * n_kv_head + head) * page_size + slot) * HD
  const size_t kv_stride = (size_t)n_kv_head * page_size * HD;
  const bf16* head_base = cache + (size_t)hk * page_size * HD;
  auto load_kv = [&](int tile, int buf) {
    const int j0 = tile * PF_BN;
    for (int c = tid; c < PF_BN * CHUNKS; c += PF_THREADS) {
      const int r = c / CHUNKS, piece = c % CHUNKS;
      const int j = j0 + r;
      bool valid = j <= pos_last;
      const bf16* src = cache;
      if (valid) {
        const int page = table[page_size == 16 ? (j >> 4) : j / page_size];
        if (page < 0 || page >= n_pages) {
          valid = false;
          if (j >= key_lo) *status = NIB_STATUS_BAD_PAGE;  // pages behind a window may be gone, and are not read
        } else {
          const int slot = page_size == 16 ? (j & 15) : j % page_size;
          src = head_base + (size_t)page * 2 * kv_stride + (size_t)slot * HD + piece * 8;
        }
      }
      cp_async16(ks + (buf * PF_BN + r) * LD + piece * 8, src, valid);
      cp_async16(vs + (buf * PF_BN + r) * LD + piece * 8, src + kv_stride, valid);
    }
  };
  load_kv(tile_first, 0);
  cp_async_commit();

  // accumulators: this thread holds rows (lane / 4) and (lane / 4 + 8) of its warp's 16
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  const int rg = warp & 3, kh = warp >> 2;                  // row group and part of the keys
  const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;        // rows within the tile
  const int p0 = pos_first + r0, p1 = pos_first + r1;       // their positions
  const int lo0 = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const int lo1 = (window > 0 && p1 - window + 1 > 0) ? p1 - window + 1 : 0;
  uint32_t qf[HD / 16][4];
  const float scale2 = scale * 1.4426950408889634f;

  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int buf = (tile - tile_first) & 1;
    if (tile < tile_last) load_kv(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();          // everything but the newest group has landed: Q and this tile
    __syncthreads();
    if (tile == tile_first) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
    }
    const bf16* kt = ks + (buf * PF_BN + kh * PF_WN) * LD;   // this warp's keys of the tile
    const bf16* vt = vs + (buf * PF_BN + kh * PF_WN) * LD;

    // ---- S = Q K^T : 16 rows x PF_WN keys per warp
    float s[PF_WN / 8][4];
#pragma unroll
    for (int i = 0; i < PF_WN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
      for (int nn = 0; nn < PF_WN / 16; ++nn) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (nn * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
        mma_bf16(s[2 * nn], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * nn + 1], qf[kk], b[2], b[3]);
      }
    }
    // ---- mask, online softmax.  Scores are kept times log2(e), so that the exponentials are plain
    // powers of two; only the tiles on the causal edge (or a window's edge) need the mask.
    const int wp0 = pos_first + rg * 16, wp1 = wp0 + 15;     // positions of the warp's rows
    const int wj0 = tile * PF_BN + kh * PF_WN;               // the warp's first key of the tile
    const bool edge = wj0 + PF_WN - 1 > wp0 || (window > 0 && wj0 < wp1 - window + 1);
    if (edge) {
      const int j_base = wj0 + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < PF_WN / 8; ++i) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = j_base + i * 8 + c;
          if (!(j <= p0 && j >= lo0)) s[i][c] = -INFINITY;
          if (!(j <= p1 && j >= lo1)) s[i][2 + c] = -INFINITY;
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < PF_WN / 8; ++i) {
      mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
      mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0 * scale2), mn1 = fmaxf(m1, mx1 * scale2);   // (scale2 > 0)
    // a row with no key yet (all masked so far) keeps m = -inf; 2^(-inf - -inf) is avoided
    const float ms0 = (mn0 == -INFINITY) ? 0.0f : mn0, ms1 = (mn1 == -INFINITY) ? 0.0f : mn1;
    const float c0 = pow2(m0 - ms0), c1 = pow2(m1 - ms1);
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int i = 0; i < PF_WN / 8; ++i) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        s[i][c] = pow2(fmaf(s[i][c], scale2, -ms0));
        s[i][2 + c] = pow2(fmaf(s[i][2 + c], scale2, -ms1));
        sum0 += s[i][c];
        sum1 += s[i][2 + c];
      }
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * c0 + sum0;
    l1 = l1 * c1 + sum1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < PF_WN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack2(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack2(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dd = 0; dd < HD / 16; ++dd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dd * 16 + 8 * (lane >> 4));
        mma_bf16(o[2 * dd], a, b[0], b[1]);
        mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();   // everyone is done with this buffer before the next load overwrites it
  }
  cp_async_wait<0>();

  // ---- the warps of a row group merge their halves (through the idle key buffers), in a fixed order
  static_assert(PF_KSPLIT == 2, "the merge below is written for two warps per row group");
  float* mo = reinterpret_cast<float*>(ks);                 // [4 row groups][32 lanes][HD / 2 + 4]
  constexpr int MO = HD / 2 + 4;
  float* mine = mo + (size_t)(rg * 32 + lane) * MO;
  if (kh == 1) {
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
    *reinterpret_cast<float4*>(mine + HD / 2) = make_float4(m0, m1, l0, l1);
  }
  __syncthreads();
  if (kh == 1) return;
  {
    const float4 other = *reinterpret_cast<const float4*>(mine + HD / 2);
    const float mn0 = fmaxf(m0, other.x), mn1 = fmaxf(m1, other.y);
    const float ms0 = (mn0 == -INFINITY) ? 0.0f : mn0, ms1 = (mn1 == -INFINITY) ? 0.0f : mn1;
    const float a0 = pow2(m0 - ms0), a1 = pow2(m1 - ms1), b0 = pow2(other.x - ms0), b1 = pow2(other.y - ms1);
    l0 = l0 * a0 + other.z * b0;
    l1 = l1 * a1 + other.w * b1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const float4 t = *reinterpret_cast<const float4*>(mine + 4 * i);
      o[i][0] = o[i][0] * a0 + t.x * b0;
      o[i][1] = o[i][1] * a0 + t.y * b0;
      o[i][2] = o[i][2] * a1 + t.z * b1;
      o[i][3] = o[i][3] * a1 + t.w * b1;
    }
  }

  // ---- normalise and store
  const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    const int d = h * HD + i * 8 + (lane & 3) * 2;
    if (r0 < n_rows)
      *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + r0) * ldo + d) = pack2(o[i][0] * i0, o[i][1] * i0);
    if (r1 < n_rows)
      *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + r1) * ldo + d) = pack2(o[i][2] * i1, o[i][3] * i1);
  }
}

template <int HD>
static int launch_prefill(const void* q, int ldq, const void* cache, void* out, int ldo, const int* block_table,
                          int max_blocks, const int* tiles, int n_tiles, const int* entry_start,
                          const int* entry_pos0, int n_head, int n_kv_head, int page_size, int n_pages, float scale,
                          int window, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * (HD + 8) * sizeof(bf16);
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(n_head, n_tiles);
  launch_pdl(attention_prefill_kernel<HD>, dim3(grid), dim3(PF_THREADS), smem, stream, 
      (const bf16*)q, ldq, (const bf16*)cache, (bf16*)out, ldo, block_table, max_blocks, tiles, entry_start,
      entry_pos0, n_head, n_kv_head, page_size, n_pages, scale, window, status);
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

extern "C" int nib_attention_prefill_supported(int head_dim) {
  return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0;
}

// tiles: n_tiles pairs (entry, first row within the entry), 64 rows each (the last of an entry may
// be shorter).  q and out rows are the step's rows; ldq, ldo and the column offsets of the head
// must keep every head's row 16-byte aligned for q and 4-byte aligned for out.
extern "C" int nib_attention_prefill(const void* q, int ldq, const void* cache, void* out, int ldo,
                                     const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                     const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head,
                                     int head_dim, int page_size, int n_pages, float scale, int window,
                                     int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!nib_attention_prefill_supported(head_dim)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0 || !(scale > 0.0f)) return NIB_ERR_BAD_ARGUMENT;
  if ((ldq & 7) || ((uintptr_t)q & 15) || (ldo & 1) || ((uintptr_t)out & 3)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_tiles > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
#define NIB_PF_CASE(D)                                                                                         \
  case D:                                                                                                      \
    return launch_prefill<D>(q, ldq, cache, out, ldo, block_table, max_blocks, tiles, n_tiles, entry_start,    \
                             entry_pos0, n_head, n_kv_head, page_size, n_pages, scale, window, status, stream);
  switch (head_dim) {
    NIB_PF_CASE(16) NIB_PF_CASE(32) NIB_PF_CASE(48) NIB_PF_CASE(64) NIB_PF_CASE(80) NIB_PF_CASE(96)
    NIB_PF_CASE(112) NIB_PF_CASE(128)
  }
#undef NIB_PF_CASE
  return NIB_ERR_UNSUPPORTED_SIZE;
}
