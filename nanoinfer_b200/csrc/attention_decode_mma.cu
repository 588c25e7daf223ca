// Attention for single decoded tokens in bfloat16 with warp-level MMAs: the split-KV scheme of
// attention_decode.cu (one block per (row, head, split of the keys), the last block of a (row, head)
// merges the splits), with the arithmetic of a tile of 16 keys done by the tensor cores.
//
// The streaming kernel spends about 29 warp instructions per (key, head): unpacking bfloat16 pairs,
// 128 multiply-adds spread over eight lanes, the shuffles that complete each dot product.  At 64
// rows that is what bounds it (its issue slots are full at 0.7 of the memory's rate), and at 8 rows
// the same work is the difference between a context of 100 and one of 1000.  Here a warp takes 16
// keys at a time:
//   * scores: S[16 keys x 8] = K[16 x hd] . Q[hd x 8] with m16n8k16, the keys' rows as the 16-row
//     operand straight from 16-byte global loads, the query in column 0 of the other operand (the
//     other seven columns are zero: a decoded token has one query per head).  A dot product does not
//     care about the order of its terms, so a lane's 16-byte piece of a key row is dealt to the
//     fragment positions as it comes, and the query's pieces the same way;
//   * softmax: the 16 scores sit in eight lanes; four shuffles bring them to where the next
//     product wants them, scores are kept times log2(e), statistics in 32-bit;
//   * output: O^T[hd x 8] += V^T[hd x 16 keys] . P^T[16 x 8], the value rows transposed in registers
//     by `movmatrix` (8x8 tiles of 16-bit values), P rounded to bfloat16 as in the prefill kernels.
// About 60 warp instructions per 16 keys and head instead of 460.  Results: column 0 of the
// accumulators, in the lanes 0, 4, ..., 28.  The warps of a block and the splits of a (row, head)
// are merged as in the streaming kernel, in fixed orders
// (crates/metal/src/shaders/batch.metal:349-424 is the reference's split and merge pair; the
// formulas are crates/core/src/kernels/reference.rs:109-142).
//
// Head sizes: multiples of 32 up to 128; pages of a multiple of 16 positions.  Everything else,
// and the true 32-bit path, stays with the streaming kernel.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int DM_WARPS = 4;
constexpr int DM_MAX_CLUSTER = 16;  // (beyond the portable 8 the kernel is marked as taking non-portable cluster sizes)

__device__ __forceinline__ void dm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// transposes an 8x8 tile of 16-bit values held one row-pair per lane (lane i: row i / 4, columns
// 2 (i % 4) and the next)
__device__ __forceinline__ uint32_t dm_transpose(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ float dm_pow2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// partial layout as in the streaming kernel: o [row][head][split][head_dim], ml [row][head][split][2]
// (a tile's keys and values are 16 registers per 32 of head size: six blocks an SM up to 64, three beyond)
// (q, cache and out carry no __restrict__: the kernel ahead writes them; see pdl_wait in common.cuh)
// STAGES > 0: a warp's tiles pass through a ring of that many stages of its own in shared memory, filled
// by `cp.async`: STAGES tiles of keys and values are on their way while another is multiplied, at no cost
// in registers (a batch of 64 rows has one block per row and head and is bound by how many bytes are in
// flight; without the ring a warp has one tile's loads, 4 KB, in flight at a time).
template <int HD, int STAGES>
__global__ void __launch_bounds__(DM_WARPS * 32, HD <= 64 ? 6 : 3)
attention_decode_mma_kernel(const bf16* q, int ldq, const bf16* cache, float* part_o,
                            float* part_ml, bf16* out, int ldo, const int* __restrict__ block_table,
                            int max_blocks, const int* __restrict__ rows, const int* __restrict__ row_entry,
                            const int* __restrict__ positions, int n_head, int n_kv_head, int page_size,
                            int n_pages, float scale, int window, int chunk, int n_splits,
                            int* counters, int* status, int cluster_merge) {
  constexpr int HALVES = HD / 32;                    // a 16-byte piece per lane covers 32 of a row's values
  constexpr bool RING = STAGES > 0;
  constexpr int NS = RING ? STAGES : 1;
  pdl_trigger();
  __shared__ __align__(16) float wo[DM_WARPS][HD];   // the warps' unnormalised outputs
  __shared__ float wm[DM_WARPS], wl[DM_WARPS];
  __shared__ int is_last_sh;
  // When the splits of a (row, head) are the blocks of one cluster (at most eight), they hand their
  // results to the first of them through distributed shared memory instead of through global scratch,
  // an arrival counter and a second read: two trips to memory less at the end of the chain.
  // (the ring's variants keep to the portable eight: with sixteen rows here six blocks of them no longer fit an SM)
  constexpr int XC = RING ? 8 : DM_MAX_CLUSTER;
  __shared__ __align__(16) float xo[XC][HD];
  __shared__ float xml[XC][2];
  extern __shared__ __align__(16) uint8_t dm_ring[]; // RING: [warp][stage][keys | values][16 rows][HD]
  if (cluster_merge) cluster_arrive();               // met below, before the first store into another block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int fr = lane >> 2, kl = lane & 3;           // this lane's key row of a tile (and + 8), its piece of a row
  const int split = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
  // The step's tables were written before the step began and the cache below this row's position
  // belongs to earlier steps: both may be read before the kernel ahead (which writes this row's own
  // key and value, and the queries) has finished.
  const int t = rows ? rows[r] : r;
  const int pos = positions[t];
  const int* table = block_table + (size_t)row_entry[t] * max_blocks;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k_begin = lo + split * chunk;
  const int k_end = min(pos + 1, k_begin + chunk);   // exclusive
  const int hk = h / (n_head / n_kv_head);
  const size_t pidx = ((size_t)r * n_head + h) * n_splits + split;
  const bool empty = k_begin >= k_end;               // nothing in this split: the merge skips l == 0
  // tiles of 16 consecutive keys (16 divides the page size, so a tile lies in one page); this warp's
  // tiles are first_tile + warp + i * DM_WARPS
  const int first_tile = empty ? 0 : k_begin >> 4, last_tile = empty ? -1 : (k_end - 1) >> 4;
  const int n_mine = (first_tile + warp <= last_tile) ? (last_tile - first_tile - warp) / DM_WARPS + 1 : 0;
  const size_t kv_stride = (size_t)n_kv_head * page_size * HD;
  const bf16* lane_base = cache + ((size_t)hk * page_size + fr) * HD + kl * 8;

  uint4 ka[HALVES], kb[HALVES], va[HALVES], vb[HALVES];   // rows fr and fr + 8 of the tile, keys and values
  bool ok_a = false, ok_b = false;                   // whether those two keys are this split's
  bool page_ok = false;                              // whether the tile's page is one of the pool's
  auto fetch = [&](int i) {
    const int j0 = (first_tile + warp + i * DM_WARPS) << 4;
    const int page = table[j0 / page_size];
    page_ok = page >= 0 && page < n_pages;
    if (!page_ok && lane == 0) *status = NIB_STATUS_BAD_PAGE;   // recorded, never followed
    const int ja = j0 + fr, jb = j0 + fr + 8;
    ok_a = page_ok && ja >= k_begin && ja < k_end;
    ok_b = page_ok && jb >= k_begin && jb < k_end;
    const bf16* kr = lane_base + (size_t)(page_ok ? page : 0) * 2 * kv_stride + (size_t)(j0 % page_size) * HD;
#pragma unroll
    for (int hh = 0; hh < HALVES; ++hh) {
      // a key that is not this split's is all zeros: its score is masked below, and its value row must
      // not bring whatever the page holds there into the product (0 x NaN)
      ka[hh] = ok_a ? *reinterpret_cast<const uint4*>(kr + hh * 32) : make_uint4(0, 0, 0, 0);
      kb[hh] = ok_b ? *reinterpret_cast<const uint4*>(kr + 8 * HD + hh * 32) : make_uint4(0, 0, 0, 0);
      va[hh] = ok_a ? *reinterpret_cast<const uint4*>(kr + kv_stride + hh * 32) : make_uint4(0, 0, 0, 0);
      vb[hh] = ok_b ? *reinterpret_cast<const uint4*>(kr + kv_stride + 8 * HD + hh * 32) : make_uint4(0, 0, 0, 0);
    }
  };
  // ---- RING: the same tile by asynchronous copies into stage i % STAGES of this warp's ring.  A row of
  // 128 or 256 bytes starts at the same bank as the row before it: odd rows keep their 16-byte pieces
  // four places further (modulo the row), so that a fragment load of eight lanes (two rows, four
  // pieces each) touches every bank once.
  constexpr int PIECES = HD / 8;
  constexpr bool SWZ = HD % 64 == 0;
  bf16* my_ring = reinterpret_cast<bf16*>(dm_ring) + (size_t)warp * NS * 2 * 16 * HD;
  uint32_t stage_ok = 0;                             // bit s: the page of stage s is one of the pool's
  auto issue = [&](int i) {
    const int j0 = (first_tile + warp + i * DM_WARPS) << 4;
    const int page = table[j0 / page_size];
    const bool pok = page >= 0 && page < n_pages;
    if (!pok && lane == 0) *status = NIB_STATUS_BAD_PAGE;       // recorded, never followed
    stage_ok = (stage_ok & ~(1u << (i % NS))) | ((pok ? 1u : 0u) << (i % NS));
    const bf16* src = cache + ((size_t)(pok ? page : 0) * 2 * n_kv_head + hk) * page_size * HD +
                      (size_t)(j0 % page_size) * HD;
    bf16* dst = my_ring + (size_t)(i % NS) * 2 * 16 * HD;
#pragma unroll
    for (int idx = lane; idx < 16 * PIECES; idx += 32) {
      const int row = idx / PIECES, pc = idx % PIECES;
      const int j = j0 + row;
      const bool ok = pok && j >= k_begin && j < k_end;         // (a key that is not this split's: zeros)
      const int ps = SWZ ? (pc ^ ((row & 1) * 4)) : pc;
      cp_async16(dst + row * HD + ps * 8, src + (size_t)row * HD + pc * 8, ok);
      cp_async16(dst + (16 + row) * HD + ps * 8, src + kv_stride + (size_t)row * HD + pc * 8, ok);
    }
    cp_async_commit();
  };
  // the stage's fragments: this lane's pieces of the rows fr and fr + 8
  auto take = [&](int i) {
    const bf16* st = my_ring + (size_t)(i % NS) * 2 * 16 * HD;
    page_ok = (stage_ok >> (i % NS)) & 1u;
#pragma unroll
    for (int hh = 0; hh < HALVES; ++hh) {
      const int pc = kl + 4 * hh;
      const int ps = SWZ ? (pc ^ ((fr & 1) * 4)) : pc;
      ka[hh] = *reinterpret_cast<const uint4*>(st + fr * HD + ps * 8);
      kb[hh] = *reinterpret_cast<const uint4*>(st + (fr + 8) * HD + ps * 8);
      va[hh] = *reinterpret_cast<const uint4*>(st + (16 + fr) * HD + ps * 8);
      vb[hh] = *reinterpret_cast<const uint4*>(st + (24 + fr) * HD + ps * 8);
    }
  };
  // none of the first tiles' keys is the one that the kernel ahead writes: they may be asked for now
  const bool early = n_mine > 0 && (((first_tile + warp) << 4) + 15) < pos;
  int issued = 0;
  if (RING) {
    while (issued < NS && issued < n_mine && (((first_tile + warp + issued * DM_WARPS) << 4) + 15) < pos) issue(issued++);
  } else if (early) {
    fetch(0);
  }
  pdl_wait();
  if (cluster_merge) cluster_wait();                 // every block of the cluster runs by now
  if (RING) {
    while (issued < NS && issued < n_mine) issue(issued++);
  }

  if (empty) {
    if (threadIdx.x == 0 && n_splits > 1) {
      if (cluster_merge) {
        store_to_rank(&xml[split][0], 0, -INFINITY);
        store_to_rank(&xml[split][1], 0, 0.0f);
      } else {
        part_ml[2 * pidx] = -INFINITY;
        part_ml[2 * pidx + 1] = 0.0f;
      }
    }
  } else {
    // the query in column 0 of the 8-column operand: the lanes 0..3 hold its pieces, the others zeros
    uint4 qf[HALVES];
#pragma unroll
    for (int hh = 0; hh < HALVES; ++hh)
      qf[hh] = fr == 0 ? *reinterpret_cast<const uint4*>(q + (size_t)t * ldq + h * HD + hh * 32 + kl * 8)
                       : make_uint4(0, 0, 0, 0);
    float acc[2 * HALVES][4];                        // O^T tiles: 16 of a row's values by 8 columns each
#pragma unroll
    for (int a = 0; a < 2 * HALVES; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.0f;
    // scores are kept times log2(e), so that the exponentials are plain powers of two
    const float scale2 = scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.0f;

    for (int i = 0; i < n_mine; ++i) {
      if (RING) {
        // tile i has landed (the issued - 1 - i tiles after it may still be on their way)
        const int behind = issued - 1 - i;
        if (NS >= 4 && behind >= 3) cp_async_wait<3>();
        else if (NS >= 3 && behind == 2) cp_async_wait<2>();
        else if (behind == 1) cp_async_wait<1>();
        else cp_async_wait<0>();
        __syncwarp();
        take(i);
      } else if (i > 0 || !early) {
        fetch(i);
      }
      const int j0 = (first_tile + warp + i * DM_WARPS) << 4;
      // ---- S = K . q: column 0 comes out in the lanes with kl == 0, c[0] for key fr and c[2] for key fr + 8
      float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int hh = 0; hh < HALVES; ++hh) {
        dm_mma(s, ka[hh].x, kb[hh].x, ka[hh].y, kb[hh].y, qf[hh].x, qf[hh].y);
        dm_mma(s, ka[hh].z, kb[hh].z, ka[hh].w, kb[hh].w, qf[hh].z, qf[hh].w);
      }
      // ---- the scores go where the next product wants P: lane kl (of every row group alike) takes the
      // keys 2 kl, 2 kl + 1, 2 kl + 8 and 2 kl + 9 of the tile
      float p[4];
      p[0] = __shfl_sync(0xffffffffu, s[0], 8 * kl);
      p[1] = __shfl_sync(0xffffffffu, s[0], 8 * kl + 4);
      p[2] = __shfl_sync(0xffffffffu, s[2], 8 * kl);
      p[3] = __shfl_sync(0xffffffffu, s[2], 8 * kl + 4);
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + 2 * kl + (e & 1) + (e >> 1) * 8;
        p[e] = (page_ok && j >= k_begin && j < k_end) ? p[e] * scale2 : -INFINITY;
        mx = fmaxf(mx, p[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m, mx);
      if (m_new != -INFINITY) {                      // (the same in every lane; else: no key of this split so far)
        const float corr = dm_pow2(m - m_new);         // (2^-inf = 0 for the first keys)
        m = m_new;
        float sum = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = dm_pow2(p[e] - m);                    // 0 for a key that is not there
          sum += p[e];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l = l * corr + sum;
#pragma unroll
        for (int a = 0; a < 2 * HALVES; ++a) {
          acc[a][0] *= corr;
          acc[a][2] *= corr;
        }
        // ---- O^T += V^T . P^T: P in column 0 (the lanes 0..3 hold it), the value rows transposed in registers.
        // Register x of a lane's piece holds the values 8 kl + 2 x (+1) of a 32-wide part of the row: the four
        // lanes' registers x make an 8x8 tile whose column 2 kl + e stands for that value.  Tiles x = 0, 1 give
        // the 16 rows of one product, tiles 2, 3 those of the next.
        const uint32_t pb0 = fr == 0 ? dm_pack(p[0], p[1]) : 0u;
        const uint32_t pb1 = fr == 0 ? dm_pack(p[2], p[3]) : 0u;
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh) {
          dm_mma(acc[2 * hh], dm_transpose(va[hh].x), dm_transpose(va[hh].y), dm_transpose(vb[hh].x),
                 dm_transpose(vb[hh].y), pb0, pb1);
          dm_mma(acc[2 * hh + 1], dm_transpose(va[hh].z), dm_transpose(va[hh].w), dm_transpose(vb[hh].z),
                 dm_transpose(vb[hh].w), pb0, pb1);
        }
      }
      if (RING && issued < n_mine) {                 // the stage that was just used takes the tile STAGES further on
        __syncwarp();
        issue(issued++);
      }
    }
    // ---- column 0 of the accumulators: lane 4 f (kl == 0) holds, in tile a = 2 hh + u, c[0] for the row
    // f of tile x = 2 u and c[2] for the row f of tile x = 2 u + 1; row f of tile x is the value
    // 32 hh + 8 (f / 2) + 2 x + f % 2 of the head
    if (kl == 0) {
#pragma unroll
      for (int a = 0; a < 2 * HALVES; ++a) {
        const int hh = a >> 1, u = a & 1;
        const int d0 = 32 * hh + 8 * (fr >> 1) + (fr & 1);
        wo[warp][d0 + 2 * (2 * u)] = acc[a][0];
        wo[warp][d0 + 2 * (2 * u + 1)] = acc[a][2];
      }
    }
    if (lane == 0) {
      wm[warp] = m;
      wl[warp] = l;
    }
    __syncthreads();
    // ---- the warps' results are merged in warp order
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) M = fmaxf(M, wm[w]);
    float L = 0.0f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) L += (wm[w] == -INFINITY) ? 0.0f : wl[w] * dm_pow2(wm[w] - M);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
      float o = 0.0f;
#pragma unroll
      for (int w = 0; w < DM_WARPS; ++w) o += (wm[w] == -INFINITY) ? 0.0f : wo[w][d] * dm_pow2(wm[w] - M);
      if (n_splits == 1)
        out[(size_t)t * ldo + h * HD + d] = __float2bfloat16_rn(L > 0.0f ? o / L : 0.0f);
      else if (cluster_merge)
        store_to_rank(&xo[split][d], 0, o);
      else
        part_o[pidx * HD + d] = o;
    }
    if (n_splits > 1 && threadIdx.x == 0) {
      if (cluster_merge) {
        store_to_rank(&xml[split][0], 0, M);
        store_to_rank(&xml[split][1], 0, L);
      } else {
        part_ml[2 * pidx] = M;                       // (in the power-of-two scale)
        part_ml[2 * pidx + 1] = L;
      }
    }
  }
  if (n_splits == 1) return;
  const float* mo;    // the splits' outputs [n_splits][HD] and (maximum, sum) pairs, wherever they met
  const float* ml;
  if (cluster_merge) {
    // ---- the first block of the cluster merges the splits, in split order
    cluster_arrive();
    cluster_wait();
    if (split != 0) return;
    mo = &xo[0][0];
    ml = &xml[0][0];
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
    const size_t base = ((size_t)r * n_head + h) * n_splits;
    mo = part_o + base * HD;
    ml = part_ml + 2 * base;
  }
  float Mx = -INFINITY;
  for (int sp = 0; sp < n_splits; ++sp) Mx = fmaxf(Mx, ml[2 * sp]);
  float Lx = 0.0f;
  for (int sp = 0; sp < n_splits; ++sp) {
    const float ls = ml[2 * sp + 1];
    if (ls > 0.0f) Lx += ls * dm_pow2(ml[2 * sp] - Mx);
  }
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float o = 0.0f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float ls = ml[2 * sp + 1];
      if (ls > 0.0f) o += mo[sp * HD + d] * dm_pow2(ml[2 * sp] - Mx);
    }
    out[(size_t)t * ldo + h * HD + d] = __float2bfloat16_rn(Lx > 0.0f ? o / Lx : 0.0f);
  }
}

}  // namespace nib

using namespace nib;

// 1 if the MMA kernel takes this shape (bfloat16 only).
extern "C" int nib_attention_decode_mma_supported(int head_dim, int page_size) {
  return (head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128) && page_size > 0 &&
         page_size % 16 == 0;
}

// How many clusters of `cluster` blocks of this kernel (no ring) the device holds at once, as the runtime
// counts them (a cluster's blocks share a GPC, so it is fewer than blocks an SM x SMs / cluster); 0 if
// the head size is not taken, a negative CUDA error code if the query fails.
extern "C" int nib_attention_decode_mma_clusters(int head_dim, int cluster) {
  if (cluster < 1 || cluster > DM_MAX_CLUSTER) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, 1, 4096);
  cfg.blockDim = dim3(DM_WARPS * 32);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = cudaSuccess;
#define NIB_DM_ROOM(HD)                                                                                              \
  do {                                                                                                               \
    if (cluster > 8) {  /* a device or driver that does not take the larger sizes holds none of them */            \
      e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, 0>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1); \
      if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }                                                 \
    }                                                                                                                \
    e = cudaOccupancyMaxActiveClusters(&n, attention_decode_mma_kernel<HD, 0>, &cfg);                                \
    if (e != cudaSuccess && cluster > 8) { (void)cudaGetLastError(); return 0; }                                     \
  } while (0)
  switch (head_dim) {
    case 32: NIB_DM_ROOM(32); break;
    case 64: NIB_DM_ROOM(64); break;
    case 96: NIB_DM_ROOM(96); break;
    case 128: NIB_DM_ROOM(128); break;
    default: return 0;
  }
#undef NIB_DM_ROOM
  return e == cudaSuccess ? n : -(int)e;
}

// Arguments as for nib_attention_decode (bfloat16): scratch holds nib_attention_decode_scratch(...)
// floats and counters n_rows * n_head zeroed ints when n_splits > 1, unless `cluster` is set: then the
// 2 to 16 splits of a (row, head) run as one cluster and merge through distributed shared memory.  q, out and
// the cache layer must be 16-byte aligned with row strides that are multiples of 8 values.
extern "C" int nib_attention_decode_mma(const void* q, int ldq, const void* cache, float* scratch, void* out,
                                        int ldo, const int* block_table, int max_blocks, const int* rows,
                                        const int* row_entry, const int* positions, int n_rows, int n_head,
                                        int n_kv_head, int head_dim, int page_size, int n_pages, float scale,
                                        int window, int chunk, int n_splits, int* counters, int* status,
                                        int cluster, int ring, cudaStream_t stream) {
  if (ring != 0 && ring != 2 && ring != 3 && ring != 4) return NIB_ERR_BAD_ARGUMENT;
  if (n_rows <= 0) return 0;
  if (!nib_attention_decode_mma_supported(head_dim, page_size)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (chunk <= 0 || chunk % 16 != 0 || n_splits <= 0) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0) return NIB_ERR_BAD_ARGUMENT;
  if (n_rows > 65535 || n_head > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || (ldq & 7)) return NIB_ERR_UNSUPPORTED_SIZE;
  // cluster != 0: the splits of a (row, head) are one cluster and merge inside it (2 to 16 splits; beyond 8 without a ring)
  if (cluster && (n_splits < 2 || n_splits > DM_MAX_CLUSTER || (n_splits > 8 && ring != 0))) return NIB_ERR_BAD_ARGUMENT;
  if (n_splits > 1 && !cluster && (scratch == nullptr || counters == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)n_rows * n_head * n_splits * head_dim : nullptr;
  const dim3 grid(n_splits, n_head, n_rows), block(DM_WARPS * 32);
  // ring: the number of shared-memory stages per warp that keys and values pass through (2 to 4 tiles in flight; 0: none)
  const size_t ring_bytes = (size_t)DM_WARPS * ring * 2 * 16 * head_dim * sizeof(bf16);
  cudaError_t e = cudaSuccess;
#define NIB_DM_LAUNCH_R(HD, RING)                                                                                \
  do {                                                                                                           \
    if (RING > 0 && ring_bytes > 32 * 1024) {  /* (static shared memory counts against the 48 KB default too) */ \
      static bool attr_set = false;                                                                              \
      if (!attr_set) {                                                                                           \
        e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)ring_bytes);                                                               \
        if (e != cudaSuccess) return (int)e;                                                                     \
        attr_set = true;                                                                                         \
      }                                                                                                          \
    }                                                                                                            \
    if (cluster && n_splits > 8) {  /* (more blocks than the portable cluster size) */                          \
      static bool wide_set = false;                                                                              \
      if (!wide_set) {                                                                                           \
        e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, RING>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1); \
        if (e != cudaSuccess) return (int)e;                                                                     \
        wide_set = true;                                                                                         \
      }                                                                                                          \
    }                                                                                                            \
    e = launch_pdl_cluster(attention_decode_mma_kernel<HD, RING>, grid, block, RING > 0 ? ring_bytes : 0, stream, \
                           cluster ? n_splits : 1, (const bf16*)q, ldq, (const bf16*)cache, part_o, part_ml,     \
                           (bf16*)out, ldo, block_table, max_blocks, rows, row_entry, positions, n_head,         \
                           n_kv_head, page_size, n_pages, scale, window, chunk, n_splits, counters, status,      \
                           cluster ? 1 : 0);                                                                     \
  } while (0)
#define NIB_DM_LAUNCH(HD)                   \
  if (ring == 2) NIB_DM_LAUNCH_R(HD, 2);      \
  else if (ring == 3) NIB_DM_LAUNCH_R(HD, 3); \
  else if (ring == 4) NIB_DM_LAUNCH_R(HD, 4); \
  else NIB_DM_LAUNCH_R(HD, 0)
  switch (head_dim) {
    case 32: NIB_DM_LAUNCH(32); break;
    case 64: NIB_DM_LAUNCH(64); break;
    case 96: NIB_DM_LAUNCH(96); break;
    default: NIB_DM_LAUNCH(128); break;
  }
#undef NIB_DM_LAUNCH
#undef NIB_DM_LAUNCH_R
  if (e != cudaSuccess) return (int)e;
  NIB_LAUNCH_CHECK();
}
