// out = act(a . w^T + bias) for steps of a few rows (at most 128), in bfloat16, with warp-level MMAs.
//
// With a few rows the product is a stream of weights with a handful of multiply-adds per weight:
// the 128-row tcgen05 MMA takes its full 128 cycles however few columns it has, its set-up
// (barriers, tensor memory, descriptors) costs more than the arithmetic, and its 128-feature tiles
// leave most SMs without work.  Here a block owns 16 output features, its warps split K, every lane
// pulls weights with independent 16-byte loads that are all in flight before any is used, and the
// small warp-level MMA (m16n8k16) multiplies them with the step's rows held in shared memory.  Where
// 16-feature tiles alone would leave SMs idle (a narrow output, a long K), the blocks of a cluster
// split K between them and exchange their partial sums through distributed shared memory, each
// block finishing a share of the rows: every sum still has one fixed order.
//
// Folded in, because each is one round trip less for a decode step:
//   * the LayerNorm that stands before the product (the rows are normalised into shared memory while
//     the first weights are on their way; formula of crates/core/src/kernels/reference.rs:42-51);
//   * the bias, GELU and residual epilogues (crates/metal/src/shaders/batch.metal:94-97,148-165);
//   * the write of keys and values into the paged cache for the fused q/k/v projection
//     (batch.metal:155-164).
// A row's result does not depend on the other rows: each (row, feature) sum has its own fixed order.
#include <map>
#include <mutex>
#include <utility>

#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int SK_WARPS = 8;
constexpr int SK_MAX_ROWS = 128;
constexpr int SK_LN_REG_WIDTH = 1024;   // rows up to this wide are normalised in registers ...
constexpr int SK_LN_MAX_WIDTH = 4096;   // ... wider ones, up to this, in shared memory
constexpr int SK_MAX_SPLIT = 8;      // blocks of a cluster that split K

struct SkinnyParams {
  const bf16* a;        // [M, K] activations (null when ln_x is given)
  int lda;
  const float* ln_x;    // residual stream, normalised here
  int ln_ldx;
  const float* ln_gamma;
  const float* ln_beta;
  const int* ln_rows;
  float ln_eps;
  const bf16* w;        // [N, K]
  int ldw;
  const float* bias;
  void* out;
  int ldo, out_f32, residual, act;
  int M, N, K;
  int split, k_per;     // blocks of a cluster and the slice of K that each takes (a multiple of 32)
  int alias;            // 1: every block has one tile, and the warps' sums take the place of the rows
  // optional: features from kv_q_dim on go to the paged cache
  bf16* kv_cache;
  const int* kv_block_table;
  const int* kv_row_entry;
  const int* kv_positions;
  int kv_max_blocks, kv_q_dim, kv_heads, kv_head_dim, kv_page_size, kv_n_pages;
  int* status;
};

__device__ __forceinline__ void mma_16x8x16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__host__ __device__ inline int skinny_ldx(int k_per) { return k_per + ((32 - k_per % 64) + 64) % 64; }

// A cluster of `split` blocks owns 16 output features at a time; block r of it takes the slice
// [r * k_per, (r + 1) * k_per) of K, and its eight warps split the slice between them (warp w takes
// the 32-wide steps w, w + 8, ...), so each warp's weights are a handful of independent 16-byte
// loads that are all in flight at once.  The warps' partial sums meet in shared memory; the
// blocks' sums are then dealt out by row (row m goes to block m % split), added there in block
// order and finished by that block.  The small tensor-core shape m16n8k16 does the arithmetic:
// weights are the 16-row operand, the step's rows (8 per tile, NT tiles) the 8-column one.  A lane's
// 16-byte piece of a weight row feeds two MMAs; since a dot product does not care about the order of
// its terms, the piece's eight values are dealt to the fragment positions as they come, and the
// rows' pieces are dealt the same way.
// ROWS: the variant for steps of more than 16 rows, whose blocks each take a row block (the others keep
// the code they had without it: a decode step of 8 rows is 0.7 % longer with the offset in every index).
template <int NT, bool ROWS>
__global__ void __launch_bounds__(SK_WARPS * 32, 2)
linear_skinny_kernel(const SkinnyParams prm) {
  pdl_trigger();
  extern __shared__ __align__(16) uint8_t sk_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A block holds at most 16 rows; a step of more runs as row blocks of 16 (grid y), every block with its
  // own copy of the chain weights -> rows -> products -> sums -> epilogue, which grows with the rows it holds.
  const int row0 = ROWS ? blockIdx.y * (NT * 8) : 0;
  const int M = ROWS ? min(prm.M - row0, NT * 8) : prm.M, S = prm.split;
  const int rank = S > 1 ? cluster_rank() : 0;
  const int walker = blockIdx.x / S, n_walkers = gridDim.x / S;
  const int k0 = rank * prm.k_per;                     // this block's slice of K
  const int Ks = min(prm.K - k0, prm.k_per);
  const int n_chunks = Ks >> 3;                        // 16-byte pieces per row of the slice
  const int ldx = skinny_ldx(prm.k_per);               // padded row: pieces of 8 rows x 4 lanes hit distinct banks
  bf16* xs = reinterpret_cast<bf16*>(sk_smem);         // [NT * 8][ldx] the step's rows (rows >= M are zeros)
  // [warps][NT][32][4] the warps' partial sums: behind the rows, or (prm.alias: a block with one tile
  // only, whose rows are used up by then) in their place
  const size_t xs_bytes = (size_t)NT * 8 * ldx * sizeof(bf16), red_bytes = (size_t)SK_WARPS * NT * 128 * sizeof(float);
  float* red = reinterpret_cast<float*>(sk_smem + (prm.alias ? 0 : xs_bytes));
  // [2][split][rows of a block][16] sums of the other blocks
  float* xch = reinterpret_cast<float*>(sk_smem + (prm.alias ? (xs_bytes > red_bytes ? xs_bytes : red_bytes)
                                                             : xs_bytes + red_bytes));
  float* ln_gb = xch + 2 * NT * 128;                   // [2][K] the norm's scale and shift
  const int n_tiles = (prm.N + 15) / 16;
  const int n_steps = (n_chunks + 3) / 4;          // 32-wide steps of the slice
  const int fr = lane >> 2, kl = lane & 3;         // this lane's feature row (and +8) and piece within a step

  // ---- Before waiting for the kernel ahead: everything that does not depend on it.  The weights of
  // this block's first tile (and the norm's parameters) are asked for now, so that they travel
  // while the previous kernel is still finishing.
  uint4 wa[4], wb[4];
  {
    const int f0 = walker * 16;
    const bf16* w0 = prm.w + (size_t)min(f0 + fr, prm.N - 1) * prm.ldw + k0;
    const bf16* w1 = prm.w + (size_t)min(f0 + fr + 8, prm.N - 1) * prm.ldw + k0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = (warp + u * SK_WARPS) * 4 + kl;
      const bool ok = c < n_chunks;
      wa[u] = ok ? *reinterpret_cast<const uint4*>(w0 + c * 8) : make_uint4(0, 0, 0, 0);
      wb[u] = ok ? *reinterpret_cast<const uint4*>(w1 + c * 8) : make_uint4(0, 0, 0, 0);
    }
  }
  if (prm.ln_x != nullptr) {
    for (int i = threadIdx.x; i < prm.K / 4; i += blockDim.x) {
      reinterpret_cast<float4*>(ln_gb)[i] = reinterpret_cast<const float4*>(prm.ln_gamma)[i];
      reinterpret_cast<float4*>(ln_gb + prm.K)[i] = reinterpret_cast<const float4*>(prm.ln_beta)[i];
    }
  }
  // What the epilogue needs and the kernel ahead does not write: the first tile's bias, and for the
  // cache-writing projection the place of each row's slot (two dependent lookups in the step's
  // tables).  Asked for now, they are there when the sums are; asked for then, each would be a round
  // trip to L2 at the very end of the chain (at 32 rows: 2 sums a thread).
  constexpr int OUTS = (NT * 128 + SK_WARPS * 32 - 1) / (SK_WARPS * 32);   // sums per thread
  constexpr bool AHEAD = true;
  float bias_r[OUTS];
  float res_r[OUTS];
  long long kv_base[OUTS];   // element offset of (page, K, head 0, slot, 0) in the cache layer; -1: bad page
#pragma unroll
  for (int q = 0; q < OUTS; ++q) {
    bias_r[q] = 0.0f; res_r[q] = 0.0f; kv_base[q] = 0;
    if (AHEAD) {
      const int o = threadIdx.x + q * SK_WARPS * 32;
      const int m = o >> 4, n = walker * 16 + (o & 15);
      if (o < NT * 128 && m < M) {
        if (prm.bias != nullptr && n < prm.N) bias_r[q] = prm.bias[n];
        if (prm.kv_cache != nullptr) {
          const int pos = prm.kv_positions[row0 + m];
          const int entry = prm.kv_row_entry[row0 + m];   // (negative: a row of no request, whose keys and values are dropped)
          const int page = entry < 0 ? 0 : prm.kv_block_table[(size_t)entry * prm.kv_max_blocks + pos / prm.kv_page_size];
          kv_base[q] = entry < 0 ? -2
                       : (page < 0 || page >= prm.kv_n_pages)
                           ? -1
                           : (long long)kv_offset(page, 0, 0, pos % prm.kv_page_size, prm.kv_heads, prm.kv_page_size,
                                                  prm.kv_head_dim);
        }
      }
    }
  }
  if (S > 1) cluster_arrive();   // met before the first exchange: by then every block of the cluster runs
  pdl_wait();
  // the residual stream's old values, asked for as early as the kernel ahead allows
  auto fetch_residual = [&](int f0) {
    if (AHEAD && prm.residual) {
#pragma unroll
      for (int q = 0; q < OUTS; ++q) {
        const int o = threadIdx.x + q * SK_WARPS * 32;
        const int m = o >> 4, n = f0 + (o & 15);
        if (o < NT * 128 && m < M && n < prm.N && (S == 1 || m % S == rank))
          res_r[q] = ((const float*)prm.out)[(size_t)(row0 + m) * prm.ldo + n];
      }
    }
  };
  fetch_residual(walker * 16);

  // ---- the step's rows into shared memory as bfloat16 (normalised on the way if asked)
  for (int i = threadIdx.x; i < (NT * 8 - M) * (ldx / 8); i += blockDim.x)   // rows past the step: zeros
    reinterpret_cast<uint4*>(xs + (size_t)M * ldx)[i] = make_uint4(0, 0, 0, 0);
  if (prm.ln_x != nullptr && prm.K > SK_LN_REG_WIDTH) {
    // Rows too wide for a lane's registers: a warp brings its row into a buffer of its own in shared
    // memory (summing on the way) and makes the other two passes there.
    __syncthreads();   // the norm's parameters are in place
    const int K = prm.K;
    float* mine = ln_gb + 2 * K + (size_t)warp * K;
    for (int m = warp; m < M; m += SK_WARPS) {
      const float* src = prm.ln_x + (size_t)(prm.ln_rows ? prm.ln_rows[row0 + m] : row0 + m) * prm.ln_ldx;
      float sum = 0.0f;
      for (int k = lane * 4; k < K; k += 128) {
        const float4 t = *reinterpret_cast<const float4*>(src + k);
        *reinterpret_cast<float4*>(mine + k) = t;
        sum += (t.x + t.y) + (t.z + t.w);
      }
      const float mean = warp_sum(sum) / (float)K;
      float sq = 0.0f;
      for (int k = lane * 4; k < K; k += 128) {   // (a lane reads back what it wrote)
        const float4 t = *reinterpret_cast<const float4*>(mine + k);
        const float d0 = t.x - mean, d1 = t.y - mean, d2 = t.z - mean, d3 = t.w - mean;
        sq += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
      const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + prm.ln_eps);
      for (int k = lane * 4; k < K; k += 128) {
        const float4 t = *reinterpret_cast<const float4*>(mine + k);
        const float4 g = *reinterpret_cast<const float4*>(ln_gb + k);
        const float4 b = *reinterpret_cast<const float4*>(ln_gb + K + k);
        uint2 packed;
        packed.x = pack2((t.x - mean) * rstd * g.x + b.x, (t.y - mean) * rstd * g.y + b.y);
        packed.y = pack2((t.z - mean) * rstd * g.z + b.z, (t.w - mean) * rstd * g.w + b.w);
        *reinterpret_cast<uint2*>(xs + (size_t)m * ldx + k) = packed;
      }
    }
  } else if (prm.ln_x != nullptr) {
    __syncthreads();   // the norm's parameters are in place
    const int K = prm.K;
    for (int m = warp; m < M; m += SK_WARPS) {
      const float* src = prm.ln_x + (size_t)(prm.ln_rows ? prm.ln_rows[row0 + m] : row0 + m) * prm.ln_ldx;
      // one read of the row into registers (K <= 1024: 32 floats a lane), then two passes on them
      float v[32];
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = (j * 32 + lane) * 4;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < K) t = *reinterpret_cast<const float4*>(src + k);
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        sum += (t.x + t.y) + (t.z + t.w);
      }
      const float mean = warp_sum(sum) / (float)K;
      float sq = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = (j * 32 + lane) * 4;
        if (k < K) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float d = v[4 * j + e] - mean;
            sq += d * d;
          }
        }
      }
      const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + prm.ln_eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = (j * 32 + lane) * 4;
        if (k < K) {
          const float4 g = *reinterpret_cast<const float4*>(ln_gb + k);
          const float4 b = *reinterpret_cast<const float4*>(ln_gb + K + k);
          __nv_bfloat162 lo = __floats2bfloat162_rn((v[4 * j] - mean) * rstd * g.x + b.x,
                                                    (v[4 * j + 1] - mean) * rstd * g.y + b.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v[4 * j + 2] - mean) * rstd * g.z + b.z,
                                                    (v[4 * j + 3] - mean) * rstd * g.w + b.w);
          uint2 packed;
          packed.x = *reinterpret_cast<uint32_t*>(&lo);
          packed.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(xs + (size_t)m * ldx + k) = packed;
        }
      }
    }
  } else {
    // asynchronous copies: all of a thread's pieces are in flight at once (a loop of loads and stores
    // was a chain of round trips; each warp bringing in only the columns of its own steps, and waiting
    // for those alone, measured the same)
    for (int m = warp; m < M; m += SK_WARPS)
      for (int c = lane; c < n_chunks; c += 32)
        cp_async16(xs + (size_t)m * ldx + c * 8, prm.a + (size_t)(row0 + m) * prm.lda + k0 + c * 8, true);
    cp_async_commit();
    cp_async_wait<0>();
  }
  __syncthreads();

  const int rows_per_rank = NT * 8 / S;
  int round = 0;
  for (int tile = walker; tile < n_tiles; tile += n_walkers, ++round) {
    const int f0 = tile * 16;
    const bf16* w0 = prm.w + (size_t)min(f0 + fr, prm.N - 1) * prm.ldw + k0;
    const bf16* w1 = prm.w + (size_t)min(f0 + fr + 8, prm.N - 1) * prm.ldw + k0;
    if (AHEAD && round > 0) {   // (the first tile's were asked for above)
#pragma unroll
      for (int q = 0; q < OUTS; ++q) {
        const int o = threadIdx.x + q * SK_WARPS * 32;
        const int n = f0 + (o & 15);
        if (o < NT * 128 && (o >> 4) < M && prm.bias != nullptr && n < prm.N) bias_r[q] = prm.bias[n];
      }
      fetch_residual(f0);
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    // this warp's steps, four at a time: eight independent 16-byte loads in flight
    for (int s0 = warp; s0 < n_steps; s0 += 4 * SK_WARPS) {
      if (s0 != warp) {   // a tile's first batch was asked for ahead: before the wait, or during the tile before
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = (s0 + u * SK_WARPS) * 4 + kl;
          const bool ok = c < n_chunks;
          wa[u] = ok ? *reinterpret_cast<const uint4*>(w0 + c * 8) : make_uint4(0, 0, 0, 0);
          wb[u] = ok ? *reinterpret_cast<const uint4*>(w1 + c * 8) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = (s0 + u * SK_WARPS) * 4 + kl;
        if ((s0 + u * SK_WARPS) < n_steps) {   // uniform over the warp
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            uint4 xb = make_uint4(0, 0, 0, 0);
            if (c < n_chunks) xb = *reinterpret_cast<const uint4*>(xs + (size_t)(t * 8 + fr) * ldx + c * 8);
            mma_16x8x16(acc[t], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xb.x, xb.y);
            mma_16x8x16(acc[t], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xb.z, xb.w);
          }
        }
      }
    }
    if (tile + n_walkers < n_tiles) {   // the next tile's first batch travels while this one is finished
      const int g0 = (tile + n_walkers) * 16;
      const bf16* v0 = prm.w + (size_t)min(g0 + fr, prm.N - 1) * prm.ldw + k0;
      const bf16* v1 = prm.w + (size_t)min(g0 + fr + 8, prm.N - 1) * prm.ldw + k0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = (warp + u * SK_WARPS) * 4 + kl;
        const bool ok = c < n_chunks;
        wa[u] = ok ? *reinterpret_cast<const uint4*>(v0 + c * 8) : make_uint4(0, 0, 0, 0);
        wb[u] = ok ? *reinterpret_cast<const uint4*>(v1 + c * 8) : make_uint4(0, 0, 0, 0);
      }
    }
    // ---- the warps' partial sums meet in shared memory and are added in warp order
    __syncthreads();   // the previous tile's sums have been read
#pragma unroll
    for (int t = 0; t < NT; ++t)
      *reinterpret_cast<float4*>(red + ((size_t)(warp * NT + t) * 32 + lane) * 4) =
          make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    __syncthreads();
    // sum o belongs to row o / 16 of the step and feature f0 + o % 16 (consecutive threads: consecutive features)
    float total[OUTS];
#pragma unroll
    for (int q = 0; q < OUTS; ++q) {
      const int o = threadIdx.x + q * SK_WARPS * 32;
      total[q] = 0.0f;
      if (o < NT * 128) {
        const int m = o >> 4, nl = o & 15;
        const int t = m >> 3, l = (nl & 7) * 4 + ((m & 7) >> 1), i = (nl >> 3) * 2 + (m & 1);
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) total[q] += red[((size_t)(w * NT + t) * 32 + l) * 4 + i];
      }
    }
    float* xb = xch + (round & 1) * NT * 128;
    if (S > 1) {
      // Row m is finished by block m % S: the others send their sums there.  Two buffers by turns:
      // a block writes into a buffer again only after the barrier of the round between, which its
      // owner reaches after reading it.
      if (round == 0) cluster_wait();
#pragma unroll
      for (int q = 0; q < OUTS; ++q) {
        const int o = threadIdx.x + q * SK_WARPS * 32;
        if (o < NT * 128) {
          const int m = o >> 4, nl = o & 15;
          const int owner = m % S;
          if (owner != rank) store_to_rank(xb + ((size_t)rank * rows_per_rank + m / S) * 16 + nl, owner, total[q]);
        }
      }
      cluster_arrive();
      cluster_wait();
    }
#pragma unroll
    for (int q = 0; q < OUTS; ++q) {
      const int o = threadIdx.x + q * SK_WARPS * 32;
      if (o >= NT * 128) continue;
      const int m = o >> 4, nl = o & 15;
      const int n = f0 + nl;
      if (n >= prm.N || m >= M) continue;
      float x = total[q];
      if (S > 1) {
        if (m % S != rank) continue;
        x = 0.0f;
        for (int r = 0; r < S; ++r)   // in block order, this block's own sum at its place
          x += (r == rank) ? total[q] : xb[((size_t)r * rows_per_rank + m / S) * 16 + nl];
      }
      x += AHEAD ? bias_r[q] : (prm.bias ? prm.bias[n] : 0.0f);
      if (prm.act == ACT_GELU_TANH) {
        float th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        x = 0.5f * x * (1.0f + th);
      } else if (prm.act == ACT_GELU_ERF) {
        x = gelu_erf(x);
      }
      if (prm.kv_cache != nullptr && n >= prm.kv_q_dim) {
        const int kv_dim = prm.kv_heads * prm.kv_head_dim;
        const int rem = n - prm.kv_q_dim;
        const int which = rem / kv_dim, head = (rem % kv_dim) / prm.kv_head_dim, d = rem % prm.kv_head_dim;
        long long base;
        if (AHEAD) {
          base = kv_base[q];
        } else {
          const int pos = prm.kv_positions[row0 + m];
          const int entry = prm.kv_row_entry[row0 + m];
          const int page = entry < 0 ? 0 : prm.kv_block_table[(size_t)entry * prm.kv_max_blocks + pos / prm.kv_page_size];
          base = entry < 0 ? -2
                 : (page < 0 || page >= prm.kv_n_pages)
                     ? -1
                     : (long long)kv_offset(page, 0, 0, pos % prm.kv_page_size, prm.kv_heads, prm.kv_page_size,
                                            prm.kv_head_dim);
        }
        if (base == -2) {
          // (a row of no request)
        } else if (base < 0) {
          *prm.status = NIB_STATUS_BAD_PAGE;
        } else {   // from (page, K, head 0, slot): K|V and the head are whole strides further
          prm.kv_cache[base + ((long long)which * prm.kv_heads + head) * prm.kv_page_size * prm.kv_head_dim + d] =
              __float2bfloat16_rn(x);
        }
      } else if (prm.out_f32) {
        float* dst = (float*)prm.out + (size_t)(row0 + m) * prm.ldo + n;
        *dst = prm.residual ? (AHEAD ? res_r[q] : *dst) + x : x;
      } else {
        ((bf16*)prm.out)[(size_t)(row0 + m) * prm.ldo + n] = __float2bfloat16_rn(x);
      }
    }
  }
  if (S > 1 && round == 0) cluster_wait();   // (a block without a tile still completes the opening barrier)
}

// 8-row MMA tiles a block holds (one or two), and the row blocks of 16 that a step of more rows is cut into
// (grid y).  Measured in whole decode steps against blocks of 32 and of 64 rows: 24 to 64 rows of GPT-2
// small take 8 to 12 % less a step in blocks of 16 than in blocks of 32, which took 9 % less than blocks of
// 64 at 64 rows; blocks of 8 are slower again from 12 rows on.
static int skinny_tiles(int M) { return M <= 8 ? 1 : 2; }
static int skinny_row_blocks(int M) { const int r = skinny_tiles(M) * 8; return (M + r - 1) / r; }

static size_t skinny_smem(int NT, int k_per, int K, bool ln, bool alias = false) {
  const size_t xs = (size_t)NT * 8 * skinny_ldx(k_per) * sizeof(bf16), red = (size_t)SK_WARPS * NT * 128 * sizeof(float);
  // (the other blocks' sums of a split K, kept without a split too: without them a decode step measured 1 % longer;
  // with the norm: its scale and shift, and for wide rows a buffer per warp)
  return (alias ? (xs > red ? xs : red) : xs + red) + (size_t)2 * NT * 128 * sizeof(float) +
         (ln ? (size_t)(2 + (K > SK_LN_REG_WIDTH ? SK_WARPS : 0)) * K * sizeof(float) : 0);
}

constexpr size_t SK_SMEM_LIMIT = 200 * 1024;
constexpr size_t SK_SMEM_TWO_PER_SM = 110 * 1024;

static int skinny_k_per(int K, int split) { return (((K + split - 1) / split) + 31) / 32 * 32; }

// How many blocks split K.  An exchange through the cluster costs about a microsecond, so K is split
// only while every block keeps at least 768 of it and no SM gets more than two blocks; and where the
// rows would not fit in shared memory otherwise.
static int skinny_split(int M, int N, int K, bool ln) {
  if (ln) return 1;   // the norm needs whole rows
  const int NT = skinny_tiles(M), n_tiles = (N + 15) / 16;
  int split = 1;
  while (split < SK_MAX_SPLIT) {
    const int s2 = split * 2, kp = skinny_k_per(K, s2);
    if ((s2 - 1) * kp >= K) break;
    const bool too_big = skinny_smem(NT, skinny_k_per(K, split), K, false) > SK_SMEM_LIMIT;
    if (!too_big && (n_tiles * s2 > 2 * 148 || kp < 768)) break;
    split = s2;
  }
  return split;
}

template <int NT, bool ROWS>
static int launch_skinny(SkinnyParams prm, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<NT, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)SK_SMEM_LIMIT);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(SK_WARPS * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  const int cluster = prm.split;   // the blocks that split K
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 2 : 1;
  // One wave: at most two blocks per SM (one when the rows take much shared memory), each cluster
  // then walks several tiles with the rows in place.  How many clusters the device holds at once is
  // asked of the runtime (a cluster's blocks share a GPC, so it is fewer than SMs / blocks): a
  // cluster too many would wait for a whole wave to end.
  int err = 0;
  auto clusters_at_once = [&](size_t smem) {
    const int per_sm = smem <= SK_SMEM_TWO_PER_SM ? 2 : 1;
    if (cluster == 1) return per_sm * 148;
    static std::mutex mu;
    static std::map<std::pair<int, size_t>, int> held;   // (blocks of a cluster, shared memory) -> clusters at once
    std::lock_guard<std::mutex> lock(mu);
    auto it = held.find({cluster, smem});
    if (it == held.end()) {
      int n = 0;
      cudaLaunchConfig_t q = cfg;
      q.gridDim = dim3(cluster * 148);
      q.dynamicSmemBytes = smem;
      q.attrs = attr + 1;      // the query takes the cluster shape only
      q.numAttrs = 1;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, linear_skinny_kernel<NT, ROWS>, &q);
      if (e != cudaSuccess) { err = (int)e; return 0; }
      if (n < 1) { err = NIB_ERR_UNSUPPORTED_SIZE; return 0; }
      it = held.emplace(std::make_pair(cluster, smem), n).first;
    }
    const int cap = it->second;
    return cap < per_sm * 148 / cluster ? cap : per_sm * 148 / cluster;
  };
  const int n_tiles = (prm.N + 15) / 16;
  const bool ln = prm.ln_x != nullptr;
  size_t smem = skinny_smem(NT, prm.k_per, prm.K, ln);
  const int row_blocks = skinny_row_blocks(prm.M);   // (every walker is there once per row block)
  auto per_row_block = [&](int c) { return c / row_blocks > 0 ? c / row_blocks : 1; };
  int cap = per_row_block(clusters_at_once(smem));
  if (err) return err;
  prm.alias = 0;
  if (n_tiles > cap) {
    // More tiles than one wave of blocks: if a block has one tile only, its warps' sums can lie where
    // the rows were, and the smaller blocks may all fit at once.
    const size_t smem_one = skinny_smem(NT, prm.k_per, prm.K, ln, true);
    const int cap_one = smem_one < smem ? per_row_block(clusters_at_once(smem_one)) : 0;
    if (err) return err;
    if (n_tiles <= cap_one) { prm.alias = 1; smem = smem_one; cap = cap_one; }
  }
  // as many walkers as the device holds at once: with 300 tiles for 296 places most blocks then have one tile
  // and four have two, where 150 blocks of two tiles each left half of the places empty (GPT-2 XL's q/k/v
  // projection; a decode step at batch 8: 2.28 -> 2.17 ms)
  const int walkers = n_tiles < cap ? n_tiles : cap;
  cfg.dynamicSmemBytes = smem;
  cfg.gridDim = dim3(walkers * prm.split, row_blocks);
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_skinny_kernel<NT, ROWS>, prm);
  if (e != cudaSuccess) return (int)e;
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

// 1 if the few-rows kernel takes this problem (ln: with the LayerNorm folded in).
extern "C" int nib_linear_skinny_supported(int M, int K, int ldw, int ln, const void* w) {
  if (M < 1 || M > SK_MAX_ROWS || K < 8 || (K & 7) || (ldw & 7) || ((uintptr_t)w & 15)) return 0;
  if (ln && (K > SK_LN_MAX_WIDTH || (K & 3))) return 0;
  const int split = skinny_split(M, 16, K, ln != 0);   // (the split that smem alone asks for)
  if (skinny_smem(skinny_tiles(M), skinny_k_per(K, split), K, ln != 0) > SK_SMEM_LIMIT) return 0;
  return 1;
}

// The product for steps of at most 128 rows (bfloat16 weights and activations; out bfloat16 or
// float32).  Options as for nib_linear_tc_small: ln_x != null folds the LayerNorm before the product
// in (`a` ignored); cache != null sends the features from q_dim on to the paged
// cache.  split: blocks of a cluster that split K (0: chosen here; 1, 2, 4 or 8).
extern "C" int nib_linear_skinny(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                                 void* out, int ldo, int M, int N, int K, int act, int residual, const float* ln_x,
                                 int ln_ldx, const float* ln_gamma, const float* ln_beta, float ln_eps,
                                 const int* ln_rows, void* cache, const int* block_table, int max_blocks,
                                 const int* row_entry, const int* positions, int q_dim, int n_kv_head,
                                 int head_dim, int page_size, int n_pages, int split, int* status,
                                 cudaStream_t stream) {
  if (N <= 0 || M <= 0) return 0;
  const bool ln = ln_x != nullptr;
  if (!nib_linear_skinny_supported(M, K, ldw, ln, w)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (!ln && a == nullptr) return NIB_ERR_BAD_ARGUMENT;
  if (residual && out_dtype != DT_F32) return NIB_ERR_BAD_ARGUMENT;
  if (cache != nullptr && (out_dtype != DT_BF16 || residual || N != q_dim + 2 * n_kv_head * head_dim))
    return NIB_ERR_BAD_ARGUMENT;
  if (split == 0) split = skinny_split(M, N, K, ln);
  if (split != 1 && split != 2 && split != 4 && split != 8) return NIB_ERR_BAD_ARGUMENT;
  if (ln && split != 1) return NIB_ERR_BAD_ARGUMENT;
  const int k_per = skinny_k_per(K, split);
  if ((split - 1) * k_per >= K) return NIB_ERR_BAD_ARGUMENT;   // a block would have nothing
  if (skinny_smem(skinny_tiles(M), k_per, K, ln) > SK_SMEM_LIMIT) return NIB_ERR_UNSUPPORTED_SIZE;
  SkinnyParams prm;
  prm.a = (const bf16*)a; prm.lda = lda;
  prm.ln_x = ln_x; prm.ln_ldx = ln_ldx; prm.ln_gamma = ln_gamma; prm.ln_beta = ln_beta; prm.ln_rows = ln_rows;
  prm.ln_eps = ln_eps;
  prm.w = (const bf16*)w; prm.ldw = ldw; prm.bias = bias; prm.out = out; prm.ldo = ldo;
  prm.out_f32 = out_dtype == DT_F32; prm.residual = residual; prm.act = act;
  prm.M = M; prm.N = N; prm.K = K; prm.split = split; prm.k_per = k_per;
  prm.kv_cache = (bf16*)cache; prm.kv_block_table = block_table; prm.kv_row_entry = row_entry;
  prm.kv_positions = positions; prm.kv_max_blocks = max_blocks; prm.kv_q_dim = q_dim; prm.kv_heads = n_kv_head;
  prm.kv_head_dim = head_dim; prm.kv_page_size = page_size; prm.kv_n_pages = n_pages;
  prm.status = status;
  if ((lda & 7) || (a != nullptr && ((uintptr_t)a & 15))) return NIB_ERR_UNSUPPORTED_SIZE;
  if (ln && ((ln_ldx & 3) || ((uintptr_t)ln_x & 15) || ((uintptr_t)ln_gamma & 15) || ((uintptr_t)ln_beta & 15)))
    return NIB_ERR_UNSUPPORTED_SIZE;
  switch (skinny_tiles(M)) {
    case 1: return launch_skinny<1, false>(prm, stream);
    default: return M > 16 ? launch_skinny<2, true>(prm, stream) : launch_skinny<2, false>(prm, stream);
  }
}
