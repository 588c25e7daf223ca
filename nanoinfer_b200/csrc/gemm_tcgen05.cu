// out = act(a . w^T + bias) in bfloat16 on the 5th-generation tensor cores (sm_100a):
// TMA loads into 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor
// memory, tcgen05.ld back to registers for a fused epilogue (bias, GELU, residual add).
//
// Both operands are K-major ([rows, K], K contiguous): activations a [M, K] and weights w [N, K],
// the "out, in" layout the reference transposes to at load (crates/core/src/weights.rs:1-9), so
// out = a . w^T is the reference's matmul (crates/core/src/kernels/reference.rs:26-37).  The tile
// that feeds the MMA's M side ("P", 128 rows) and the one that feeds its N side ("Q", 16..256
// rows) are interchangeable:
//   * P = activations, Q = weights: from 17 rows on (one padded row tile up to 128 rows);
//   * P = weights, Q = activations ("swap-AB"): every weight byte is read exactly once and the few
//     rows still fill the 128-row MMA; for at most 16 rows, for the options below, and up to 128
//     rows where the 128-feature tiles alone fill the device (the head).
//
// One CTA computes one P x Q tile: warp 0 issues the TMA loads, warp 1 allocates tensor memory
// and issues the MMAs, warps 2..5 run the epilogue (each owns the 32 TMEM lanes of its quarter).
// The epilogue writes the finished tile into the (by then idle) pipeline buffers and hands it
// to TMA: a tiled store, or for the residual sum a tiled reduce-add, so that x += tile happens in
// the L2 without the SM reading x.  Outputs whose pitch or address TMA cannot take (rows not a
// multiple of 16 bytes) are written with plain stores instead.
// In the swapped orientation two more things can be folded in.  The activations may be given as the
// 32-bit residual stream plus LayerNorm parameters: the four epilogue warps, idle until the MMAs
// finish, normalise the rows and write them as the MMA's bfloat16 operand straight into shared
// memory while the weights are still on their way, which saves a kernel and a round trip per norm.
// And K may be split over several blocks whose partial tiles are summed by the last one to finish,
// so that a product with few output tiles still pulls its weights with the whole GPU.
// Every wait on an mbarrier is bounded: if it runs out, the kernel records
// NIB_STATUS_WAIT_TIMEOUT, stops issuing work, frees its tensor memory and returns.
#include <cuda.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"


namespace nib {

constexpr int TC_BP = 128;        // rows of the P tile = MMA M
constexpr int TC_BK = 64;         // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_THREADS = 192;

struct TcParams {
  int p_rows, q_rows, K;
  int bq;            // rows of the Q tile = MMA N (multiple of 16, at most 256)
  int stages;
  int k_sub;         // 64-wide K blocks per pipeline stage (1 or 2)
  int kb_per_split;  // 64-wide K blocks per split of K (grid.z splits; their tiles are summed by reduce-add)
  int swap;          // 0: P = activations (out[p, q]); 1: P = weights (out[q, p])
  void* out;
  int ldo;
  int out_f32;
  const float* bias;
  int act;
  int residual;
  int tma_store;     // 1: the epilogue stages the tile in shared memory and stores it with TMA
  int* status;
  // Optional (swapped orientation only): output features from q_dim on are keys and values, which go
  // straight to their slots in the paged cache instead of to `out` (the reference's QKV epilogue,
  // crates/metal/src/shaders/batch.metal:155-164)
  bf16* kv_cache;
  const int* kv_block_table;
  const int* kv_row_entry;
  const int* kv_positions;
  int kv_max_blocks, kv_q_dim, kv_heads, kv_head_dim, kv_page_size, kv_n_pages;
  // Optional (swapped orientation only): the activations are LayerNorm(x[rows]) computed by the block
  // itself from the 32-bit residual stream, instead of a bfloat16 matrix loaded by TMA
  // (reference formula: crates/core/src/kernels/reference.rs:42-51)
  const float* ln_x;
  const float* ln_gamma;
  const float* ln_beta;
  const int* ln_rows;
  int ln_ldx;
  float ln_eps;
  // Optional (swapped orientation only): K split over grid.z with the partial tiles summed, in split
  // order, by the block of a tile that finishes last (for outputs that cannot be reduce-added)
  float* fix_partials;
  int* fix_counters;
  int fix_splits;
};

// The epilogue's activation.  The result is rounded to bfloat16 (8 bits of mantissa), so the tanh
// form uses the hardware tanh (relative error about 2^-11); the erf form keeps the accurate erff.
template <int ACT>
__device__ __forceinline__ float epilogue_act(float u) {
  if (ACT == ACT_GELU_TANH) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (u + 0.044715f * u * u * u)));
    return 0.5f * u * (1.0f + t);
  }
  if (ACT == ACT_GELU_ERF) return gelu_erf(u);
  return u;
}
// ------------------------------------------------------------------ the kernel
// ACT is a template parameter so that each instantiation carries the code of its own activation only
// (the unrolled epilogue would otherwise hold dozens of copies of erff).
template <int ACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                 const __grid_constant__ CUtensorMap map_o, const TcParams prm) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  // tiles must start on a 1024-byte boundary for the 128-byte swizzle
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[TC_MAX_STAGES];
  __shared__ uint64_t empty_bar[TC_MAX_STAGES];
  __shared__ uint64_t tmem_full_bar;
  __shared__ uint64_t q_ready_bar;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ int epi_ok_sh[4];
  __shared__ __align__(16) float bias_sh[256];   // the bias of the tile's columns (plain orientation)
  __shared__ int fix_last_sh;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = prm.stages, bq = prm.bq;
  const int k_sub = prm.k_sub;
  const bool ln = prm.ln_x != nullptr;            // the Q operand is made here, not loaded
  const uint32_t p_bytes = TC_BP * TC_BK * 2, q_bytes = (uint32_t)bq * TC_BK * 2;  // one 64-wide block each
  // a stage holds k_sub blocks of P and, unless Q is resident, of Q; multiples of 1024 (bq % 16 == 0)
  const uint32_t stage_bytes = (uint32_t)k_sub * (p_bytes + (ln ? 0u : q_bytes));
  const int p0 = blockIdx.x * TC_BP, q0 = blockIdx.y * bq;
  // this block's share of K, in 64-wide blocks, and in pipeline stages
  const int kb_begin = blockIdx.z * prm.kb_per_split;
  const int kb_end = min((prm.K + TC_BK - 1) / TC_BK, kb_begin + prm.kb_per_split);
  const int num_kb = (kb_end - kb_begin + k_sub - 1) / k_sub;
  const bool first_split = blockIdx.z == 0;
  uint8_t* q_region = smem + (size_t)stages * stage_bytes;   // resident Q blocks (LayerNorm mode)
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < bq) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    mbar_init(&q_ready_bar, 128);
    abort_sh = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_p) : "memory");
    if (!ln) asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_q) : "memory");
    if (prm.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_o) : "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_base_sh, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  volatile int* abort_flag = &abort_sh;
  // Only the producer goes on before the kernel ahead has finished: it asks for the WEIGHT tiles of
  // the first stages (they do not depend on that kernel), and waits before it asks for activations.
  if (warp != 0) pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer.  Issuing a stage costs one thread several hundred cycles (a wait,
    // an expect and the copies, each a dependent instruction), so up to four lanes issue in
    // parallel: lane l takes the stage steps l, l + L, ... (the same instructions on different
    // barriers and buffers, so the lanes run in lockstep).
    const int L = stages < 4 ? stages : 4;
    const bool weights_are_p = prm.swap != 0;
    // first round (the stages are all free): the weight tiles now, the activation tiles after the wait
    const int first_round = num_kb < stages ? num_kb : stages;
    if (lane < L) {
      for (int kb = lane; kb < first_round; kb += L) {
        uint8_t* sp = smem + (size_t)kb * stage_bytes;
        mbar_expect_tx(&full_bar[kb], stage_bytes);
        for (int sub = 0; sub < k_sub; ++sub) {
          const int kb64 = kb_begin + kb * k_sub + sub;
          const int kx = (kb64 < kb_end ? kb64 : (prm.K + TC_BK - 1) / TC_BK) * TC_BK;
          if (weights_are_p) tma_load_2d(sp + sub * p_bytes, &map_p, &full_bar[kb], kx, p0);
          else tma_load_2d(sp + k_sub * p_bytes + sub * q_bytes, &map_q, &full_bar[kb], kx, q0);
        }
      }
    }
    __syncwarp();
    pdl_wait();
    if (lane < L) {
      for (int kb = lane; kb < first_round; kb += L) {
        uint8_t* sp = smem + (size_t)kb * stage_bytes;
        for (int sub = 0; sub < k_sub; ++sub) {
          const int kb64 = kb_begin + kb * k_sub + sub;
          const int kx = (kb64 < kb_end ? kb64 : (prm.K + TC_BK - 1) / TC_BK) * TC_BK;
          if (!weights_are_p) tma_load_2d(sp + sub * p_bytes, &map_p, &full_bar[kb], kx, p0);
          else if (!ln) tma_load_2d(sp + k_sub * p_bytes + sub * q_bytes, &map_q, &full_bar[kb], kx, q0);
        }
      }
      // later rounds: a stage is refilled when the MMAs have read it
      for (int kb = first_round + lane; kb < num_kb; kb += L) {
        const int s = kb % stages;
        const uint32_t parity = ((kb / stages) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[s], parity, abort_flag)) break;
        uint8_t* sp = smem + (size_t)s * stage_bytes;
        mbar_expect_tx(&full_bar[s], stage_bytes);
        for (int sub = 0; sub < k_sub; ++sub) {
          // a block past this split's end is asked for past the end of K: it arrives as zeros
          const int kb64 = kb_begin + kb * k_sub + sub;
          const int kx = (kb64 < kb_end ? kb64 : (prm.K + TC_BK - 1) / TC_BK) * TC_BK;
          tma_load_2d(sp + sub * p_bytes, &map_p, &full_bar[s], kx, p0);
          if (!ln) tma_load_2d(sp + k_sub * p_bytes + sub * q_bytes, &map_q, &full_bar[s], kx, q0);
        }
      }
    }
    __syncwarp();
    if (*abort_flag && lane == 0) {
      // give copies that are still in flight time to land before the block's shared memory goes away
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) {
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer: lane 0 waits and issues.  One thread runs a dependent
    // instruction every few cycles, so the loop is kept to the bare minimum: the high half of the
    // matrix descriptors is a constant, the low half is the stage's address plus a small offset.
    const uint32_t idesc = umma_idesc(TC_BP, bq);
    const uint32_t desc_hi = (uint32_t)(umma_desc(0) >> 32);
    const uint32_t desc_lo0 = (uint32_t)umma_desc(smem_u32(smem));   // address field: bits 0..13, in 16-byte units
    const uint32_t stage_step = stage_bytes >> 4, p_step = p_bytes >> 4, q_step = q_bytes >> 4;
    const uint32_t q_off = (uint32_t)k_sub * p_step;
    const uint32_t q_res0 = (uint32_t)umma_desc(smem_u32(q_region));
    int s = 0;
    uint32_t parity = 0, lo_stage = desc_lo0, accumulate = 0;
    bool ok = true;
    if (ln) ok = warp_mbar_wait(&q_ready_bar, 0, abort_flag, lane);  // the normalised rows are in place
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      if (!warp_mbar_wait(&full_bar[s], parity, abort_flag, lane)) break;
      tc_fence_after();
      if (lane == 0) {
        for (int sub = 0; sub < k_sub; ++sub) {
          const uint32_t pa = lo_stage + sub * p_step;
          const uint32_t qa = ln ? q_res0 + (uint32_t)(kb * k_sub + sub) * q_step : lo_stage + q_off + sub * q_step;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // 16 bf16 = 32 bytes = 2 address units further along K inside the swizzled row
            uint64_t da, db;
            asm("mov.b64 %0, {%1, %2};" : "=l"(da) : "r"(pa + 2 * k), "r"(desc_hi));
            asm("mov.b64 %0, {%1, %2};" : "=l"(db) : "r"(qa + 2 * k), "r"(desc_hi));
            umma_bf16(tmem_base, da, db, idesc, accumulate);
            accumulate = 1;
          }
        }
        umma_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
      }
      lo_stage += stage_step;
      if (++s == stages) {
        s = 0;
        parity ^= 1;
        lo_stage = desc_lo0;
      }
    }
    if (lane == 0) {
      umma_commit(&tmem_full_bar);  // arrives when every MMA above has finished
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps: warp w owns TMEM lanes 32 * (w % 4) .. +32
    const int quarter = warp & 3;
    const int pl = quarter * 32 + lane;      // this thread's row within the P tile
    const int p = p0 + pl;
    if (ln) {
      // While the weights travel: normalise this tile's rows and lay them down as the resident Q
      // operand, [local K block][row][64 bf16] in the 128-byte swizzle.  One warp per row at a time.
      const int ew = warp - 2;
      const int K = prm.K;
      const int n_local = kb_end - kb_begin;
      const int n_blocks = num_kb * k_sub;   // blocks the MMAs will read (the tail ones are zeros)
      for (int r = ew; r < bq; r += 4) {
        const int m = q0 + r;
        const bool valid = m < prm.q_rows;
        float mean = 0.0f, rstd = 0.0f;
        const float* src = prm.ln_x;
        if (valid) {
          src = prm.ln_x + (size_t)(prm.ln_rows ? prm.ln_rows[m] : m) * prm.ln_ldx;
          float sum = 0.0f;
          for (int k = lane; k < K; k += 32) sum += src[k];
          mean = warp_sum(sum) / (float)K;
          float sq = 0.0f;
          for (int k = lane; k < K; k += 32) {
            const float d = src[k] - mean;
            sq += d * d;
          }
          rstd = 1.0f / sqrtf(warp_sum(sq) / (float)K + prm.ln_eps);
        }
        for (int i = 0; i < n_blocks; ++i) {
          const int k = (kb_begin + i) * TC_BK + lane * 2;
          float v0 = 0.0f, v1 = 0.0f;
          if (valid && i < n_local) {
            if (k < K) v0 = (src[k] - mean) * rstd * prm.ln_gamma[k] + prm.ln_beta[k];
            if (k + 1 < K) v1 = (src[k + 1] - mean) * rstd * prm.ln_gamma[k + 1] + prm.ln_beta[k + 1];
          }
          uint8_t* dst = q_region + (size_t)i * q_bytes + (size_t)r * 128 + (((lane >> 2) ^ (r & 7)) << 4) + (lane & 3) * 4;
          *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMAs
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&q_ready_bar)) : "memory");
    }
    // While the MMAs run: the bias of this tile's columns into shared memory.  (Read from global
    // memory in the epilogue, every 16 columns would stall for a round trip to L2 of their own: the
    // four epilogue warps have nothing to hide it behind.)
    if (!prm.swap) {
      for (int c = (int)threadIdx.x - 64; c < bq; c += 128)
        bias_sh[c] = (prm.bias && first_split && q0 + c < prm.q_rows) ? prm.bias[q0 + c] : 0.0f;
    }
    // the four epilogue warps go on only if all of them saw the accumulator complete
    if (lane == 0) epi_ok_sh[quarter] = mbar_wait(&tmem_full_bar, 0, abort_flag) ? 1 : 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = (epi_ok_sh[0] & epi_ok_sh[1] & epi_ok_sh[2] & epi_ok_sh[3]) != 0;
    tc_fence_after();
    const bool p_ok = p < prm.p_rows;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);

    if (ok && !prm.swap) {
      // ======== plain orientation: this thread owns row p, the columns are output features ========
      if (prm.tma_store) {
        // Every MMA has finished, so every pipeline buffer is idle: the tile is staged there in blocks
        // of [128 rows][128 bytes] in the 128-byte swizzle.  64 columns at a time: four
        // tensor-memory loads in flight, one wait.
        for (int g0 = 0; g0 < bq; g0 += 64) {
          uint32_t raw[4][16];
          const int n_sub = min(4, (bq - g0) / 16);  // uniform over the block
#pragma unroll
          for (int sub = 0; sub < 4; ++sub)
            if (sub < n_sub) tmem_ld16_issue(lane_addr + (uint32_t)(g0 + sub * 16), raw[sub]);
          tmem_ld_wait();
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (sub >= n_sub) continue;
            const int c0 = g0 + sub * 16;
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(raw[sub][j]);
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(bias_sh + c0 + j);
              v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
            }
            if (ACT != ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = epilogue_act<ACT>(v[j]);
            }
            if (prm.out_f32) {
              uint8_t* blk = smem + (size_t)(c0 / 32) * 16384 + (size_t)pl * 128;
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                const int chunk = ((c0 % 32 + j) / 4) ^ (pl & 7);
                *reinterpret_cast<float4*>(blk + chunk * 16) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            } else {
              uint8_t* blk = smem + (size_t)(c0 / 64) * 16384 + (size_t)pl * 128;
#pragma unroll
              for (int j = 0; j < 16; j += 8) {
                const int chunk = ((c0 % 64 + j) / 8) ^ (pl & 7);
                *reinterpret_cast<uint4*>(blk + chunk * 16) =
                    make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                               pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
              }
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to TMA
        asm volatile("bar.sync 1, 128;" ::: "memory");                // the four epilogue warps
        if (warp == 2 && lane == 0) {
          const int cols = prm.out_f32 ? 32 : 64;
          for (int c = 0; c < bq && q0 + c < prm.q_rows; c += cols) {
            const void* src = smem + (size_t)(c / cols) * 16384;
            if (prm.residual) tma_reduce_add_2d(&map_o, src, q0 + c, p0);
            else tma_store_2d(&map_o, src, q0 + c, p0);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory may go away now
        }
      } else {
        // out[p, q0 + c0 + j] with plain stores: this thread writes 16 consecutive features of its row
        for (int c0 = 0; c0 < bq; c0 += 16) {
          if (q0 + c0 >= prm.q_rows) break;  // uniform over the warp
          float v[16];
          tmem_ld16(lane_addr + (uint32_t)c0, v);
          if (!p_ok) continue;
          const int n0 = q0 + c0;
          const int nv = min(16, prm.q_rows - n0);
#pragma unroll
          for (int j = 0; j < 16; ++j) {  // unrolled with a guard: v[] must stay in registers
            if (j < nv) {
              const float x = epilogue_act<ACT>(v[j] + bias_sh[c0 + j]);
              if (prm.out_f32) {
                float* o = (float*)prm.out + (size_t)p * prm.ldo + n0 + j;
                *o = prm.residual ? *o + x : x;
              } else {
                ((bf16*)prm.out)[(size_t)p * prm.ldo + n0 + j] = __float2bfloat16_rn(x);
              }
            }
          }
        }
      }
    } else if (ok) {
      // ======== swapped orientation: this thread owns output feature p, the columns are tokens ========
      bool is_last = true;
      if (prm.fix_splits > 1) {
        // K was split: park the raw partial tile, and let the block that arrives last add them up
        const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
        float* mine = prm.fix_partials + ((tile * prm.fix_splits + blockIdx.z) * bq) * TC_BP;
        for (int c0 = 0; c0 < bq; c0 += 16) {
          if (q0 + c0 >= prm.q_rows) break;
          float v[16];
          tmem_ld16(lane_addr + (uint32_t)c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(size_t)(c0 + j) * TC_BP + pl] = v[j];
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int arrived = atomicAdd(&prm.fix_counters[tile], 1);
          fix_last_sh = arrived == prm.fix_splits - 1;
          if (fix_last_sh) prm.fix_counters[tile] = 0;  // zero again for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        is_last = fix_last_sh != 0;
        if (is_last) __threadfence();
      }
      if (is_last) {
        const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
        const bool add_bias = prm.bias != nullptr && p_ok && (first_split || prm.fix_splits > 1);
        const float bias_p = add_bias ? prm.bias[p] : 0.0f;
        const bool to_cache = prm.kv_cache != nullptr && p >= prm.kv_q_dim;
        int kv_which = 0, kv_head = 0, kv_d = 0;
        if (to_cache) {
          const int kv_dim = prm.kv_heads * prm.kv_head_dim;
          const int rem = p - prm.kv_q_dim;
          kv_which = rem / kv_dim;
          kv_head = (rem % kv_dim) / prm.kv_head_dim;
          kv_d = rem % prm.kv_head_dim;
        }
        for (int c0 = 0; c0 < bq; c0 += 16) {
          if (!prm.tma_store && q0 + c0 >= prm.q_rows) break;  // uniform over the warp
          float v[16];
          if (prm.fix_splits > 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            if (q0 + c0 < prm.q_rows) {
              for (int z = 0; z < prm.fix_splits; ++z) {   // in split order: the sum is the same every run
                const float* part = prm.fix_partials + ((tile * prm.fix_splits + z) * bq + c0) * TC_BP + pl;
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += part[(size_t)j * TC_BP];
              }
            }
          } else {
            tmem_ld16(lane_addr + (uint32_t)c0, v);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = q0 + c0 + j;
            const float x = epilogue_act<ACT>(v[j] + bias_p);
            if (prm.tma_store) {
              // a dense [tokens][128 features] tile in the idle pipeline buffers, lanes along the features
              if (prm.out_f32)
                reinterpret_cast<float*>(smem)[(c0 + j) * TC_BP + pl] = x;
              else
                reinterpret_cast<bf16*>(smem)[(c0 + j) * TC_BP + pl] = __float2bfloat16_rn(x);
            } else if (m < prm.q_rows && p_ok) {
              if (to_cache) {
                const int pos = prm.kv_positions[m];
                const int entry = prm.kv_row_entry[m];
                const int page = entry < 0 ? 0 : prm.kv_block_table[(size_t)entry * prm.kv_max_blocks +
                                                                    pos / prm.kv_page_size];
                if (entry < 0) {
                  // (a row of no request: its keys and values are dropped)
                } else if (page < 0 || page >= prm.kv_n_pages) {
                  *prm.status = NIB_STATUS_BAD_PAGE;
                } else {
                  prm.kv_cache[kv_offset(page, kv_which, kv_head, pos % prm.kv_page_size, prm.kv_heads,
                                         prm.kv_page_size, prm.kv_head_dim) + kv_d] = __float2bfloat16_rn(x);
                }
              } else if (prm.out_f32) {
                float* o = (float*)prm.out + (size_t)m * prm.ldo + p;
                *o = prm.residual ? *o + x : x;
              } else {
                ((bf16*)prm.out)[(size_t)m * prm.ldo + p] = __float2bfloat16_rn(x);
              }
            }
          }
        }
        if (prm.tma_store) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to TMA
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 2 && lane == 0) {
            if (prm.residual) tma_reduce_add_2d(&map_o, smem, p0, q0);
            else tma_store_2d(&map_o, smem, p0, q0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory may go away now
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0 && abort_sh) *prm.status = NIB_STATUS_WAIT_TIMEOUT;
}

// ------------------------------------------------------------------ host side
}  // namespace nib

using namespace nib;

// 1 if the tensor-core path takes this problem, 0 if the caller must use the SIMT kernel.
// `a` may be null (activations made in the kernel by LayerNorm): then only the weights are checked.
extern "C" int nib_linear_tc_supported(const void* a, int lda, const void* w, int ldw, int K) {
  if (K < 8 || (K & 7) || (ldw & 7)) return 0;  // TMA: 16-byte row strides
  if ((uintptr_t)w & 15) return 0;
  if (a != nullptr && ((lda & 7) || ((uintptr_t)a & 15))) return 0;
  return 1;
}

struct KvTarget {
  void* cache;
  const int* block_table;
  const int* row_entry;
  const int* positions;
  int max_blocks, q_dim, heads, head_dim, page_size, n_pages;
};
struct LnSource {
  const float* x;
  int ldx;
  const float* gamma;
  const float* beta;
  float eps;
  const int* rows;
};
struct FixScratch {
  float* partials;
  long long n_floats;
  int* counters;
  int n_counters;
};

constexpr int TC_LN_MAX_Q_BYTES = 96 * 1024;  // resident normalised activations in LayerNorm mode

static int launch_tc(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                     int ldo, int M, int N, int K, int act, int residual, const LnSource* ln, const KvTarget* kv,
                     const FixScratch* fix, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (ln != nullptr) a = nullptr;
  if (ln == nullptr && a == nullptr) return NIB_ERR_BAD_ARGUMENT;
  if (!nib_linear_tc_supported(a, lda, w, ldw, K)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (residual && out_dtype != DT_F32) return NIB_ERR_BAD_ARGUMENT;
  if (ln != nullptr && M > 128) return NIB_ERR_UNSUPPORTED_SIZE;
  TcParams prm;
  prm.K = K;
  prm.out = out;
  prm.ldo = ldo;
  prm.out_f32 = out_dtype == DT_F32;
  prm.bias = bias;
  prm.act = act;
  prm.residual = residual;
  prm.status = status;
  prm.kv_cache = nullptr;
  prm.kv_block_table = prm.kv_row_entry = prm.kv_positions = nullptr;
  prm.kv_max_blocks = prm.kv_q_dim = prm.kv_heads = prm.kv_head_dim = prm.kv_page_size = prm.kv_n_pages = 0;
  if (kv != nullptr) {
    if (M > 128 || out_dtype != DT_BF16 || act != ACT_NONE || residual) return NIB_ERR_BAD_ARGUMENT;
    if (N != kv->q_dim + 2 * kv->heads * kv->head_dim) return NIB_ERR_BAD_ARGUMENT;
    prm.kv_cache = (bf16*)kv->cache;
    prm.kv_block_table = kv->block_table;
    prm.kv_row_entry = kv->row_entry;
    prm.kv_positions = kv->positions;
    prm.kv_max_blocks = kv->max_blocks; prm.kv_q_dim = kv->q_dim; prm.kv_heads = kv->heads;
    prm.kv_head_dim = kv->head_dim; prm.kv_page_size = kv->page_size; prm.kv_n_pages = kv->n_pages;
  }
  prm.ln_x = nullptr; prm.ln_gamma = prm.ln_beta = nullptr; prm.ln_rows = nullptr; prm.ln_ldx = 0; prm.ln_eps = 0.0f;
  if (ln != nullptr) {
    prm.ln_x = ln->x; prm.ln_ldx = ln->ldx; prm.ln_gamma = ln->gamma; prm.ln_beta = ln->beta;
    prm.ln_eps = ln->eps; prm.ln_rows = ln->rows;
  }
  prm.fix_partials = nullptr; prm.fix_counters = nullptr; prm.fix_splits = 0;
  // Weights on the MMA's M side ("swap") for the fewest rows, for the options that need it, and where its
  // 128-feature tiles alone fill the device (the head); else activations on the M side even for 17 to 128
  // rows (one row tile, padded): the swapped product has N / 128 blocks, 38 for GPT-2 XL's q/k/v, the other
  // N / 64 and a split of K for the residual, and a step of an 80-token prompt takes 4.3 ms instead of 5.3.
  prm.swap = M <= 128 && (M <= 16 || kv != nullptr || ln != nullptr || fix != nullptr || (N + TC_BP - 1) / TC_BP >= 148);
  const int esz = prm.out_f32 ? 4 : 2;
  // TMA can store the tile if the output's rows are 16-byte multiples (it also clips a store at the
  // tensor's edge in 16-byte pieces, so the row length must be a multiple too)
  const bool tma_ok = ((uintptr_t)out & 15) == 0 && ((long)ldo * esz) % 16 == 0 && ((long)N * esz) % 16 == 0;
  const int num_kb64 = (K + TC_BK - 1) / TC_BK;
  const void *p_base, *q_base;
  int p_ld, q_ld, splits = 1;
  if (prm.swap) {
    prm.p_rows = N; prm.q_rows = M; p_base = w; p_ld = ldw; q_base = a; q_ld = lda;
    prm.bq = (M + 15) / 16 * 16;
    prm.tma_store = tma_ok && kv == nullptr;
    // Few tiles cannot pull the weights at full bandwidth: split K over more blocks, at least two
    // 64-wide blocks each.  The residual add sums the splits in memory (TMA reduce-add); other
    // outputs need the caller's scratch, where the last block of a tile adds the partial tiles up.
    const int tiles = (N + TC_BP - 1) / TC_BP;
    if (tiles < 148 && num_kb64 >= 4) {
      int want = (148 + tiles - 1) / tiles;
      if (want > num_kb64 / 2) want = num_kb64 / 2;
      if (want >= 2) {
        if (residual && prm.tma_store) {
          splits = want;
        } else if (fix != nullptr && fix->partials != nullptr && fix->counters != nullptr &&
                   (long long)tiles * want * prm.bq * TC_BP <= fix->n_floats && tiles <= fix->n_counters) {
          splits = want;
          prm.fix_partials = fix->partials;
          prm.fix_counters = fix->counters;
        }
      }
    }
  } else {
    prm.p_rows = M; prm.q_rows = N; p_base = a; p_ld = lda; q_base = w; q_ld = ldw;
    // Pick the Q tile (and a split of K for residual outputs) by a model of the block's time, in
    // cycles, from measurements of this kernel: a 64-wide K block costs what its operands take to
    // arrive at about 53 bytes a cycle and SM (the MMAs are faster), and a block has fixed costs
    // (set-up, the first load's latency, epilogue, store).  Up to 148 blocks run one per SM; more
    // than that run two per SM where the staged tile allows: the two share the SM's load bandwidth,
    // and one's fixed costs hide behind the other's loads.
    const int p_tiles = (M + TC_BP - 1) / TC_BP;
    double best = 1e30;
    int best_bq = 64, best_splits = 1;
    for (int bq = 256; bq >= 64; bq -= 64) {
      if (bq > 64 && N < bq) continue;
      const int tiles = p_tiles * ((N + bq - 1) / bq);
      const int max_splits = (residual && tma_ok) ? (num_kb64 >= 8 ? num_kb64 / 4 : 1) : 1;
      for (int sp = 1; sp <= max_splits && sp <= 8; ++sp) {
        const long ctas = (long)tiles * sp;
        const double kb = (double)((num_kb64 + sp - 1) / sp);
        const double load = 2.4 * (TC_BP + bq), mma = (double)bq;
        const double per_kb = load > mma ? load : mma;
        const double fixed = 3500.0 + (act != ACT_NONE ? 32.0 : 20.0) * bq;
        const bool two = ctas > 148 && (size_t)TC_BP * bq * esz <= 100 * 1024;
        double cost;
        if (!two) {
          cost = (double)((ctas + 147) / 148) * (kb * per_kb + fixed);
        } else {
          const long rounds = (ctas + 295) / 296;                  // rounds of two blocks per SM
          const bool last_single = ctas - (rounds - 1) * 296 <= 148;   // the last round has one block per SM
          cost = (double)(rounds - 1) * (2.0 * kb * per_kb + fixed) +
                 (last_single ? kb * per_kb + fixed : 2.0 * kb * per_kb + fixed);
        }
        if (cost < best) { best = cost; best_bq = bq; best_splits = sp; }
      }
    }
    prm.bq = best_bq;
    splits = best_splits;
    if (N < 64) prm.bq = (N + 15) / 16 * 16;
    prm.tma_store = tma_ok && prm.bq % 64 == 0;
    if (!prm.tma_store) splits = 1;
  }
  prm.kb_per_split = (num_kb64 + splits - 1) / splits;
  splits = (num_kb64 + prm.kb_per_split - 1) / prm.kb_per_split;
  if (prm.fix_partials != nullptr) prm.fix_splits = splits;
  if (prm.fix_splits <= 1) { prm.fix_partials = nullptr; prm.fix_counters = nullptr; prm.fix_splits = 0; }
  // A deep pipeline (one block per SM) unless the grid is several waves of blocks: then a block gets
  // about half (a third, for the many bandwidth-bound tiles of a decode step's head) of an SM's
  // shared memory, so that two or three blocks share an SM and one's prologue and epilogue hide
  // behind the others' loads and MMAs.
  const long n_ctas = (long)((prm.p_rows + TC_BP - 1) / TC_BP) * ((prm.q_rows + prm.bq - 1) / prm.bq) * splits;
  const size_t staging = prm.tma_store ? (size_t)TC_BP * prm.bq * esz : 0;
  const bool pair = !prm.swap && ln == nullptr && n_ctas > 148 && staging <= 100 * 1024;
  prm.k_sub = (!pair && prm.bq <= 128 && prm.kb_per_split >= 4) ? 2 : 1;
  const int num_stage_steps = (prm.kb_per_split + prm.k_sub - 1) / prm.k_sub;
  const int q_block = prm.bq * TC_BK * 2;
  size_t q_resident = 0;
  if (ln != nullptr) {
    q_resident = (size_t)num_stage_steps * prm.k_sub * q_block;
    if (q_resident > (size_t)TC_LN_MAX_Q_BYTES) return NIB_ERR_UNSUPPORTED_SIZE;
  }
  const int stage_bytes = prm.k_sub * (TC_BP * TC_BK * 2 + (ln != nullptr ? 0 : q_block));
  long budget = (pair ? 100 : (prm.swap && n_ctas > 2 * 148 ? 72 : 200)) * 1024 - (long)q_resident;
  if (budget < 2 * stage_bytes) budget = 2 * stage_bytes;
  int stages = (int)(budget / stage_bytes);
  if (stages < 2) stages = 2;
  if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
  if (stages > num_stage_steps) stages = num_stage_steps;
  if (stages < 1) stages = 1;
  prm.stages = stages;
  size_t tile_bytes = (size_t)stages * stage_bytes + q_resident;
  if (staging > tile_bytes) tile_bytes = staging;
  const size_t smem = tile_bytes + 1024;
  if (smem > 225 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;

  CUtensorMap map_p, map_q, map_o;
  if (!make_map(&map_p, p_base, false, prm.p_rows, K, p_ld, TC_BP, TC_BK, true)) return NIB_ERR_DRIVER;
  if (ln == nullptr) {
    if (!make_map(&map_q, q_base, false, prm.q_rows, K, q_ld, prm.bq, TC_BK, true)) return NIB_ERR_DRIVER;
  } else {
    map_q = map_p;  // unused
  }
  if (prm.tma_store) {
    const bool ok = prm.swap ? make_map(&map_o, out, prm.out_f32, M, N, ldo, prm.bq, TC_BP, false)
                             : make_map(&map_o, out, prm.out_f32, M, N, ldo, TC_BP, prm.out_f32 ? 32 : 64, true);
    if (!ok) return NIB_ERR_DRIVER;
  } else {
    map_o = map_p;  // unused
  }

  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<ACT_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         225 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(linear_tc_kernel<ACT_GELU_TANH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               225 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(linear_tc_kernel<ACT_GELU_ERF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               225 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((prm.p_rows + TC_BP - 1) / TC_BP, (prm.q_rows + prm.bq - 1) / prm.bq, splits);
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (act == ACT_GELU_TANH)
    launch_pdl(linear_tc_kernel<ACT_GELU_TANH>, grid, dim3(TC_THREADS), smem, stream, map_p, map_q, map_o, prm);
  else if (act == ACT_GELU_ERF)
    launch_pdl(linear_tc_kernel<ACT_GELU_ERF>, grid, dim3(TC_THREADS), smem, stream, map_p, map_q, map_o, prm);
  else if (act == ACT_NONE)
    launch_pdl(linear_tc_kernel<ACT_NONE>, grid, dim3(TC_THREADS), smem, stream, map_p, map_q, map_o, prm);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_linear_tc(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                             void* out, int ldo, int M, int N, int K, int act, int residual, int* status,
                             cudaStream_t stream) {
  return launch_tc(out_dtype, a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, nullptr, nullptr, nullptr,
                   status, stream);
}

// The general form for steps of at most 128 rows.  Any of three options may be on:
//   * ln_x != null: the activations are LayerNorm(ln_x[ln_rows[m] or m]) (gamma, beta, eps), made in
//     the kernel from the 32-bit residual stream (`a` is ignored);
//   * cache != null: the fused query/key/value projection: the first q_dim features go to out, the
//     rest to the rows' slots in one cache layer [n_pages, 2, n_kv_head, page_size, head_dim];
//   * fix_partials != null: scratch (floats, and zeroed int counters that the kernel leaves zero)
//     that lets K be split over blocks for outputs that are not a residual add.
// Returns NIB_ERR_UNSUPPORTED_SIZE where the shape is not taken (more than 128 rows with ln_x, or
// too much K for the resident activations); the caller then runs the plain kernels.
extern "C" int nib_linear_tc_small(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                                   void* out, int ldo, int M, int N, int K, int act, int residual,
                                   const float* ln_x, int ln_ldx, const float* ln_gamma, const float* ln_beta,
                                   float ln_eps, const int* ln_rows, void* cache, const int* block_table,
                                   int max_blocks, const int* row_entry, const int* positions, int q_dim,
                                   int n_kv_head, int head_dim, int page_size, int n_pages, float* fix_partials,
                                   long long fix_floats, int* fix_counters, int fix_n_counters, int* status,
                                   cudaStream_t stream) {
  if (M > 128) return NIB_ERR_UNSUPPORTED_SIZE;
  LnSource ln{ln_x, ln_ldx, ln_gamma, ln_beta, ln_eps, ln_rows};
  KvTarget kv{cache, block_table, row_entry, positions, max_blocks, q_dim, n_kv_head, head_dim, page_size, n_pages};
  FixScratch fix{fix_partials, fix_floats, fix_counters, fix_n_counters};
  return launch_tc(out_dtype, a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, ln_x ? &ln : nullptr,
                   cache ? &kv : nullptr, fix_partials ? &fix : nullptr, status, stream);
}

