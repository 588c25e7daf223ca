// out = act(a . w^T + bias) for many rows (prompt portions), in bfloat16, by PAIRS of thread blocks
// that share one 256-row tcgen05 MMA (cta_group::2).
//
// At a few thousand rows the single-block kernel (gemm_tcgen05.cu) is bound by how fast an SM pulls
// its operands from L2: a 128 x 256 tile needs 48 KB per 64 of K for 256 cycles of MMA.  Here two
// blocks of a cluster, on two SMs, make one 256 x N tile: each loads its own 128 rows of the
// activations and only HALF of the weight tile (N / 2 rows); the MMA, issued by the first block of
// the pair, reads the activations from each block's own shared memory and the two weight halves from
// both, and leaves each block's 128 rows of the result in that block's tensor memory.  32 KB per 64
// of K and SM instead of 48.
//
// Roles in a block: warp 0 TMA producer (the second block's loads signal the FIRST block's
// barriers), warp 1 tensor-memory allocation and, in the first block, MMA issue (its commits arrive
// at the barriers of both blocks), warps 2..5 epilogue as in the single-block kernel (bias, GELU,
// residual through TMA reduce-add, which is also how K is split over blocks).  Every wait on a
// barrier is bounded and ends in the status word.  Same formulas as gemm_tcgen05.cu
// (crates/core/src/kernels/reference.rs:26-37; epilogues crates/metal/src/shaders/batch.metal:94-97).
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace nib {

constexpr int PR_BP = 128;        // rows of a block's share of the tile (the pair makes 256)
constexpr int PR_BK = 64;         // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int PR_MAX_STAGES = 8;
constexpr int PR_THREADS = 192;

struct PairParams {
  int M, N, K;
  int bq;            // columns of the tile = MMA N (a multiple of 32, at most 256); a block loads bq / 2 weight rows
  int stages;
  int kb_per_split;  // 64-wide K blocks per split of K (grid.z splits; their tiles are summed by reduce-add)
  int out_f32;
  const float* bias;
  int residual;
  int* status;
  // Optional: output columns from kv_q_dim on are keys and values, which go straight to the rows' slots
  // in the paged cache instead of to `out` (the reference's QKV epilogue,
  // crates/metal/src/shaders/batch.metal:155-164); q_dim and head_dim are multiples of 16
  bf16* kv_cache;
  const int* kv_block_table;
  const int* kv_row_entry;
  const int* kv_positions;
  int kv_max_blocks, kv_q_dim, kv_heads, kv_head_dim, kv_page_size, kv_n_pages;
};

// ------------------------------------------------------------------ PTX wrappers of the pair forms
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives, when the MMAs issued so far are done, at the barrier at this place in BOTH blocks of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
// a tile load whose completion is counted at `bar_cluster_addr`, a barrier of the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// the address, in the cluster's shared-memory window, of `local` in block `rank`
__device__ __forceinline__ uint32_t cluster_addr_of(const void* local, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}

template <int ACT>
__device__ __forceinline__ float pair_act(float u) {
  if (ACT == ACT_GELU_TANH) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (u + 0.044715f * u * u * u)));
    return 0.5f * u * (1.0f + t);
  }
  if (ACT == ACT_GELU_ERF) return gelu_erf(u);
  return u;
}

template <int ACT>
__global__ void __launch_bounds__(PR_THREADS, 1)
linear_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_o, const PairParams prm) {
  pdl_trigger();
  extern __shared__ uint8_t pr_smem_raw[];
  // tiles must start on a 1024-byte boundary for the 128-byte swizzle (the same offset in both blocks)
  uint8_t* smem = (uint8_t*)(((uintptr_t)pr_smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[PR_MAX_STAGES];    // used in the pair's first block
  __shared__ __align__(8) uint64_t empty_bar[PR_MAX_STAGES];   // in both: the MMAs have read the stage
  __shared__ __align__(8) uint64_t tmem_full_bar;              // in both: every MMA is done
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  __shared__ int epi_ok_sh[4];
  __shared__ __align__(16) float bias_sh[256];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = cluster_rank();              // 0: the pair's first block (issues the MMAs), 1: the second
  const int stages = prm.stages, bq = prm.bq, half = bq / 2;
  const uint32_t a_bytes = PR_BP * PR_BK * 2, w_bytes = (uint32_t)half * PR_BK * 2;
  const uint32_t stage_bytes = a_bytes + w_bytes;          // a multiple of 1024 (half % 8 == 0)
  const int p0 = (blockIdx.x >> 1) * (2 * PR_BP) + rank * PR_BP;   // this block's rows
  const int q0 = blockIdx.y * bq;                                  // the tile's columns ...
  const int qh0 = q0 + rank * half;                                // ... and the weight rows this block loads
  const int kb_begin = blockIdx.z * prm.kb_per_split;
  const int kb_end = min((prm.K + PR_BK - 1) / PR_BK, kb_begin + prm.kb_per_split);
  const int num_kb = kb_end - kb_begin;
  const bool first_split = blockIdx.z == 0;
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < bq) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    abort_sh = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_o) : "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_base_sh, tmem_cols);   // one warp of each block of the pair
  tc_fence_before();
  __syncthreads();
  // both blocks' barriers are initialised before either sends a load or a commit to the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  volatile int* abort_flag = &abort_sh;
  // Only the producer goes on before the kernel ahead has finished: it asks for the WEIGHT tiles of
  // the first stages (they do not depend on that kernel), and waits before it asks for activations.
  if (warp != 0) pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer (one lane): this block's rows of the activations and its half of
    // the weight tile; completion is counted at the first block's barrier, which expects both blocks' bytes
    if (lane == 0) {
      const int first_round = num_kb < stages ? num_kb : stages;
      for (int kb = 0; kb < first_round; ++kb) {   // (the stages are all free)
        if (rank == 0) mbar_expect_tx(&full_bar[kb], 2 * stage_bytes);
        tma_load_2d_pair(smem + (size_t)kb * stage_bytes + a_bytes, &map_w, cluster_addr_of(&full_bar[kb], 0),
                         (kb_begin + kb) * PR_BK, qh0);
      }
    }
    __syncwarp();
    pdl_wait();
    if (lane == 0) {
      const int first_round = num_kb < stages ? num_kb : stages;
      for (int kb = 0; kb < first_round; ++kb)
        tma_load_2d_pair(smem + (size_t)kb * stage_bytes, &map_a, cluster_addr_of(&full_bar[kb], 0),
                         (kb_begin + kb) * PR_BK, p0);
      for (int kb = first_round; kb < num_kb; ++kb) {
        const int s = kb % stages;
        if (!mbar_wait(&empty_bar[s], ((kb / stages) & 1) ^ 1, abort_flag)) break;
        uint8_t* sp = smem + (size_t)s * stage_bytes;
        if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * stage_bytes);
        const uint32_t bar = cluster_addr_of(&full_bar[s], 0);
        const int kx = (kb_begin + kb) * PR_BK;
        tma_load_2d_pair(sp, &map_a, bar, kx, p0);
        tma_load_2d_pair(sp + a_bytes, &map_w, bar, kx, qh0);
      }
      if (*abort_flag) {
        // give copies that are still in flight time to land before the block's shared memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issue, in the pair's first block only: M = 256 over the two blocks
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = umma_idesc(2 * PR_BP, bq);
      uint32_t accumulate = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % stages;
        if (!mbar_wait(&full_bar[s], (kb / stages) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pa = smem_u32(smem + (size_t)s * stage_bytes), wa = pa + a_bytes;
#pragma unroll
        for (int k = 0; k < PR_BK / 16; ++k) {   // 16 bf16 = 32 bytes further along K inside the swizzled row
          umma_bf16_pair(tmem_base, umma_desc(pa + k * 32), umma_desc(wa + k * 32), idesc, accumulate);
          accumulate = 1;
        }
        umma_commit_pair(&empty_bar[s]);   // frees the stage, in both blocks, when these MMAs have read it
      }
      umma_commit_pair(&tmem_full_bar);     // arrives in both blocks when every MMA above has finished
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps: warp w owns tensor-memory lanes 32 * (w % 4) .. +32 = rows of this block
    const int quarter = warp & 3;
    const int pl = quarter * 32 + lane;
    for (int c = (int)threadIdx.x - 64; c < bq; c += 128)   // while the MMAs run: the bias of the tile's columns
      bias_sh[c] = (prm.bias && first_split && q0 + c < prm.N) ? prm.bias[q0 + c] : 0.0f;
    // the cache slot of this thread's row (two dependent look-ups in the step's tables), while the MMAs run
    long long kv_base = -1;   // element offset of (page, K, head 0, slot, 0) in the cache layer
    const bool kv_tile = prm.kv_cache != nullptr && q0 + bq > prm.kv_q_dim;
    if (kv_tile && p0 + pl < prm.M) {
      const int pos = prm.kv_positions[p0 + pl];
      const int entry = prm.kv_row_entry[p0 + pl];   // (negative: a row of no request, whose keys and values are dropped)
      const int page = entry < 0 ? 0 : prm.kv_block_table[(size_t)entry * prm.kv_max_blocks + pos / prm.kv_page_size];
      if (entry < 0) {}
      else if (page < 0 || page >= prm.kv_n_pages) *prm.status = NIB_STATUS_BAD_PAGE;
      else kv_base = (long long)kv_offset(page, 0, 0, pos % prm.kv_page_size, prm.kv_heads, prm.kv_page_size, prm.kv_head_dim);
    }
    if (lane == 0) epi_ok_sh[quarter] = mbar_wait(&tmem_full_bar, 0, abort_flag) ? 1 : 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = (epi_ok_sh[0] & epi_ok_sh[1] & epi_ok_sh[2] & epi_ok_sh[3]) != 0;
    tc_fence_after();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (ok) {
      // Every MMA has finished, so every pipeline buffer (of both blocks) is idle: the block's 128 rows
      // are staged in its own buffers in blocks of [128 rows][128 bytes] in the 128-byte swizzle.
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
            for (int j = 0; j < 16; ++j) v[j] = pair_act<ACT>(v[j]);
          }
          if (kv_tile && q0 + c0 >= prm.kv_q_dim) {
            // 16 consecutive values of one head of this row's key or value: 32 bytes into its cache slot
            if (kv_base >= 0 && q0 + c0 < prm.N) {
              const int kv_dim = prm.kv_heads * prm.kv_head_dim, rem = q0 + c0 - prm.kv_q_dim;
              const int which = rem / kv_dim, head = (rem % kv_dim) / prm.kv_head_dim, d = rem % prm.kv_head_dim;
              bf16* dst = prm.kv_cache + kv_base +
                          ((long long)which * prm.kv_heads + head) * prm.kv_page_size * prm.kv_head_dim + d;
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]),
                                                          pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
              *reinterpret_cast<uint4*>(dst + 8) = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]),
                                                              pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
            }
          } else if (prm.out_f32) {
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
                  make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]), pack_bf16(v[j + 4], v[j + 5]),
                             pack_bf16(v[j + 6], v[j + 7]));
            }
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to TMA
      asm volatile("bar.sync 1, 128;" ::: "memory");                // the four epilogue warps
      if (warp == 2 && lane == 0) {
        const int cols = prm.out_f32 ? 32 : 64;
        const int n_out = prm.kv_cache != nullptr ? prm.kv_q_dim : prm.N;   // columns that go to `out`
        for (int c = 0; c < bq && q0 + c < n_out; c += cols) {
          const void* src = smem + (size_t)(c / cols) * 16384;
          if (prm.residual) tma_reduce_add_2d(&map_o, src, q0 + c, p0);
          else tma_store_2d(&map_o, src, q0 + c, p0);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory may go away now
      }
    }
  }
  // Neither block frees tensor memory (the pair form frees in both) or leaves while the other still
  // reads its accumulator or may be sent a commit.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (threadIdx.x == 0 && abort_sh) *prm.status = NIB_STATUS_WAIT_TIMEOUT;
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, tmem_cols);
  }
}

}  // namespace nib

using namespace nib;

// 1 if the pair kernel takes this problem: many rows, rows of 16-byte multiples everywhere (TMA loads
// and stores), an output that TMA can store (bfloat16, or the 32-bit residual stream).
extern "C" int nib_linear_tc_pair_supported(int out_dtype, const void* a, int lda, const void* w, int ldw,
                                            const void* out, int ldo, int M, int N, int K, int residual) {
  const int esz = out_dtype == DT_F32 ? 4 : 2;
  if (M < 256 || N < 64 || K < 8 || (K & 7) || (ldw & 7) || (lda & 7)) return 0;
  if (((uintptr_t)w & 15) || ((uintptr_t)a & 15) || ((uintptr_t)out & 15)) return 0;
  if (((long)ldo * esz) % 16 != 0 || ((long)N * esz) % 16 != 0) return 0;
  if (out_dtype != DT_BF16 && out_dtype != DT_F32) return 0;
  if (residual && out_dtype != DT_F32) return 0;
  return 1;
}

template <int ACT>
static int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_o,
                       const PairParams& prm, dim3 grid, size_t smem, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_pair_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         225 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaError_t e = launch_pdl_cluster(linear_tc_pair_kernel<ACT>, grid, dim3(PR_THREADS), smem, stream, 2, map_a, map_w,
                                     map_o, prm);
  if (e != cudaSuccess) return (int)e;
  NIB_LAUNCH_CHECK();
}

// bq: columns of a tile (0: chosen here); splits: splits of K for residual outputs (0: chosen here).
// cache != null: the fused query/key/value projection: the first q_dim columns go to out, the rest to the
// rows' slots in one cache layer [n_pages, 2, n_kv_head, page_size, head_dim].
extern "C" int nib_linear_tc_pair(int out_dtype, const void* a, int lda, const void* w, int ldw, const float* bias,
                                  void* out, int ldo, int M, int N, int K, int act, int residual, int bq, int splits,
                                  void* cache, const int* block_table, int max_blocks, const int* row_entry,
                                  const int* positions, int q_dim, int n_kv_head, int head_dim, int page_size,
                                  int n_pages, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (cache != nullptr) {
    // the fused q/k/v projection: bfloat16, no residual, whole 16-value pieces of a head per thread, and a
    // tile's columns that go to `out` a multiple of what one TMA store moves
    if (out_dtype != DT_BF16 || residual || n_kv_head <= 0 || N != q_dim + 2 * n_kv_head * head_dim) return NIB_ERR_BAD_ARGUMENT;
    if ((q_dim & 63) || (head_dim & 15) || ((uintptr_t)cache & 15)) return NIB_ERR_UNSUPPORTED_SIZE;
  }
  if (!nib_linear_tc_pair_supported(out_dtype, a, lda, w, ldw, out, ldo, M, N, K, residual)) return NIB_ERR_UNSUPPORTED_SIZE;
  const int esz = out_dtype == DT_F32 ? 4 : 2;
  const int num_kb = (K + PR_BK - 1) / PR_BK;
  const int pairs = (M + 2 * PR_BP - 1) / (2 * PR_BP);
  // The tile and the split of K by a model of a block's time, in cycles, from measurements: a 64-wide K
  // block costs what its operands take to arrive (about 53 bytes a cycle and SM) or its four MMAs of
  // 128 cycles, whichever is longer, and a block has fixed costs (set-up, first load, epilogue, store).
  // Up to 148 blocks run one per SM; more run two per SM, sharing its load bandwidth while one's fixed
  // costs hide behind the other's loads.
  const bool pick_bq = bq == 0, pick_splits = splits == 0;
  if (pick_bq || pick_splits) {
    double best = 1e30;
    int best_bq = pick_bq ? 128 : bq, best_sp = pick_splits ? 1 : splits;
    for (int cand = 256; cand >= 128; cand -= 64) {
      if (!pick_bq && cand != bq) continue;
      if (pick_bq && N < cand && cand > 128) continue;
      for (int sp = 1; sp <= 8; sp *= 2) {
        if (!pick_splits && sp != splits) continue;
        if (sp > 1 && (!residual || num_kb / sp < 6)) continue;   // (a split keeps at least six K blocks)
        const long blocks = 2L * pairs * ((N + cand - 1) / cand) * sp;
        const double kb = (double)((num_kb + sp - 1) / sp);
        const double load = 2.4 * (PR_BP + cand / 2), per_kb = load > 512.0 ? load : 512.0;
        const double fixed = 3500.0 + (act != ACT_NONE ? 32.0 : 20.0) * cand;
        const bool two = blocks > 148 && (size_t)PR_BP * cand * esz <= 100 * 1024;
        double cost;
        if (!two) {
          cost = (double)((blocks + 147) / 148) * (kb * per_kb + fixed);
        } else {
          const long rounds = (blocks + 295) / 296;
          const bool last_single = blocks - (rounds - 1) * 296 <= 148;
          cost = (double)(rounds - 1) * (2.0 * kb * per_kb + fixed) +
                 (last_single ? kb * per_kb + fixed : 2.0 * kb * per_kb + fixed);
        }
        if (cost < best * (sp > 1 ? 1.0001 : 1.0)) { best = cost; best_bq = cand; best_sp = sp; }   // ties: more splits
      }
    }
    bq = best_bq;
    splits = best_sp;
  }
  if (bq < 32 || bq > 256 || bq % 32 != 0) return NIB_ERR_BAD_ARGUMENT;
  if (splits < 1 || (splits > 1 && !residual)) return NIB_ERR_BAD_ARGUMENT;
  PairParams prm;
  prm.M = M; prm.N = N; prm.K = K; prm.bq = bq;
  prm.kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + prm.kb_per_split - 1) / prm.kb_per_split;
  prm.out_f32 = out_dtype == DT_F32; prm.bias = bias; prm.residual = residual; prm.status = status;
  prm.kv_cache = (bf16*)cache; prm.kv_block_table = block_table; prm.kv_row_entry = row_entry;
  prm.kv_positions = positions; prm.kv_max_blocks = max_blocks; prm.kv_q_dim = q_dim; prm.kv_heads = n_kv_head;
  prm.kv_head_dim = head_dim; prm.kv_page_size = page_size; prm.kv_n_pages = n_pages;
  const int stage_bytes = PR_BP * PR_BK * 2 + (bq / 2) * PR_BK * 2;
  // grids of more than one wave of pairs: about half of an SM's shared memory a block, so that two
  // pairs share two SMs and one's epilogue hides behind the other's loads and MMAs
  const long n_blocks = 2L * pairs * ((N + bq - 1) / bq) * splits;
  const size_t staging0 = (size_t)PR_BP * bq * esz;
  const bool two = n_blocks > 148 && staging0 <= 100 * 1024;
  int stages = ((two ? 100 : 200) * 1024) / stage_bytes;
  if (stages > PR_MAX_STAGES) stages = PR_MAX_STAGES;
  if (stages > prm.kb_per_split) stages = prm.kb_per_split;
  if (stages < 1) stages = 1;
  prm.stages = stages;
  size_t tile_bytes = (size_t)stages * stage_bytes;
  const size_t staging = (size_t)PR_BP * bq * esz;
  if (staging > tile_bytes) tile_bytes = staging;
  const size_t smem = tile_bytes + 1024;
  CUtensorMap map_a, map_w, map_o;
  if (!make_map(&map_a, a, false, M, K, lda, PR_BP, PR_BK, true)) return NIB_ERR_DRIVER;
  if (!make_map(&map_w, w, false, N, K, ldw, bq / 2, PR_BK, true)) return NIB_ERR_DRIVER;
  if (!make_map(&map_o, out, prm.out_f32, M, N, ldo, PR_BP, prm.out_f32 ? 32 : 64, true)) return NIB_ERR_DRIVER;
  dim3 grid(2 * pairs, (N + bq - 1) / bq, splits);
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (act == ACT_GELU_TANH) return launch_pair<ACT_GELU_TANH>(map_a, map_w, map_o, prm, grid, smem, stream);
  if (act == ACT_GELU_ERF) return launch_pair<ACT_GELU_ERF>(map_a, map_w, map_o, prm, grid, smem, stream);
  if (act == ACT_NONE) return launch_pair<ACT_NONE>(map_a, map_w, map_o, prm, grid, smem, stream);
  return NIB_ERR_BAD_ARGUMENT;
}
