// Causal attention for prompt portions on the fifth-generation tensor cores: S = Q K^T and O += P V
// by tcgen05.mma with S and O in tensor memory, keys and values brought page by page by TMA.
//
// One block takes 128 consecutive query rows of one request and one head (head size 64) and walks
// the keys in tiles of 128.  Warps 0 and 6 are the TMA producers of keys and of values: their lanes
// look the tile's pages up in the request's block table and load them (16 rows x 128 bytes a load)
// into rings of three stages of 128-byte-swizzled shared memory.  Warp 1 issues the MMAs: S = Q K^T (128 x 128 x 64) into
// one of three score buffers in tensor memory, three tiles ahead of the softmax; and, once the softmax
// warps have laid P down in shared memory as bfloat16 (three buffers), O += P V (128 x 64 x 128; V is
// read as it lies, keys down the rows, as an MN-major operand), accumulated in tensor memory over
// all tiles.  Warps 2..5 are the softmax: a thread owns a row, so the row maximum and sum need no
// exchange between threads.  The running maximum is only raised when a tile exceeds it by more than
// 2^8 (P stays below 2^8, the final division by the sum is exact all the same): only then is O read
// from tensor memory, scaled and written back, which is rare after the first tiles, so the softmax
// warps normally go from one tile's scores to the next without waiting for an MMA.  Softmax in
// 32-bit with scores kept times log2(e); formula and masking as in attention_prefill.cu
// (crates/core/src/kernels/reference.rs:109-142); tiling after the reference's attn_prefill_flash
// (crates/metal/src/shaders/attn.metal:100-218).
//
// Every wait on a barrier is bounded: a wait that runs out sets the block's abort flag and the
// device status word, every role leaves its loop, tensor memory is freed, and the kernel returns.
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"


namespace nib {

constexpr int AT_BM = 128;      // query rows per block = MMA M
constexpr int AT_HD = 64;       // head size: one 128-byte swizzle row
constexpr int AT_THREADS = 224;   // keys' producer, MMA issue, four softmax warps, values' producer
constexpr int AT_UNIT = 16;     // rows of one TMA load of keys or values (divides the page size)

struct AtParams {
  const int* block_table;
  int max_blocks;
  const int* tiles;         // pairs (entry, first row within the entry), 128 rows each
  const int* entry_start;
  const int* entry_pos0;
  int n_head, n_kv_head, page_size, n_pages;
  float scale;
  int window;
  bf16* out;
  int ldo;
  int* status;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 2^x by the hardware's approximation (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float at_pow2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

constexpr int AT_STAGES = 3;     // stages of keys and values
constexpr int AT_NBUF = 3;       // score buffers in tensor memory and P buffers in shared memory
constexpr float AT_RAISE = 8.0f; // the running maximum is raised when a tile exceeds it by more than 2^8

// AT_BN: keys per tile.  64: two blocks an SM (256 columns of tensor memory and 97 KB each); 128: one
// block an SM with the whole tensor memory, half as many MMA instructions per key for the scores (an
// instruction of this shape takes about 128 cycles however narrow it is).
template <int AT_BN>
struct AtShape {
  static constexpr int KV_STAGE = AT_BN * 128;            // bytes of a stage of keys (or values): [BN keys][64]
  static constexpr int P_BYTES = (AT_BN / 64) * 16384;    // one P buffer: [BN / 64 key blocks][128 rows][64 keys]
  static constexpr uint32_t O_COL = AT_NBUF * AT_BN;      // tensor memory: the score buffers, then O
  static constexpr uint32_t TMEM_COLS = AT_BN == 64 ? 256 : 512;
  static constexpr size_t SMEM = 16384 + 2 * AT_STAGES * KV_STAGE + AT_NBUF * P_BYTES + 1024;
};

template <int AT_BN>
__global__ void __launch_bounds__(AT_THREADS, AT_BN == 64 ? 2 : 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const AtParams prm) {
  pdl_trigger();
  extern __shared__ uint8_t at_smem_raw[];
  // tiles must start on a 1024-byte boundary for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int AT_KV_STAGE = AtShape<AT_BN>::KV_STAGE, P_BYTES = AtShape<AT_BN>::P_BYTES;
  constexpr uint32_t O_COL = AtShape<AT_BN>::O_COL, TMEM_COLS = AtShape<AT_BN>::TMEM_COLS;
  uint8_t* q_s = smem;                                  // [128 rows][64]              16 KB
  uint8_t* k_s = q_s + 16384;                           // [stages][BN keys][64]
  uint8_t* v_s = k_s + AT_STAGES * AT_KV_STAGE;         // [stages][BN keys][64]
  uint8_t* p_s = v_s + AT_STAGES * AT_KV_STAGE;         // [2][BN / 64][128 rows][64 keys]
  __shared__ __align__(8) uint64_t q_full, k_full[AT_STAGES], k_empty[AT_STAGES], v_full[AT_STAGES], v_empty[AT_STAGES],
      s_full[AT_NBUF], p_full[AT_NBUF], o_full[AT_NBUF];
  __shared__ uint32_t tmem_base_sh;
  __shared__ int abort_sh;
  volatile int* abort_flag = &abort_sh;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // (heads are the fast index of the grid: blocks start in the order of the tile list, longest first)
  const int e = prm.tiles[2 * blockIdx.y], q_off = prm.tiles[2 * blockIdx.y + 1];
  const int h = blockIdx.x, hk = h / (prm.n_head / prm.n_kv_head);
  const int row0 = prm.entry_start[e] + q_off;                    // first row of the tile in the step
  const int n_rows = min(AT_BM, prm.entry_start[e + 1] - row0);
  const int pos_first = prm.entry_pos0[e] + q_off;                // position of the tile's first row
  const int pos_last = pos_first + n_rows - 1;
  const int* table = prm.block_table + (size_t)e * prm.max_blocks;
  const int window = prm.window;
  const int key_lo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int tile_first = key_lo / AT_BN, tile_last = pos_last / AT_BN;
  const int n_it = tile_last - tile_first + 1;

  if (threadIdx.x == 0) {
    abort_sh = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < AT_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < AT_NBUF; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_full[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // tensor memory: the score buffers (BN columns each), then the output O (64 columns)
  if (warp == 1) tmem_alloc(&tmem_base_sh, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sh;
  pdl_wait();   // the queries, and this step's keys and values, come from the kernels ahead

  if (warp == 0 || warp == 6) {
    // ---------------- producers: Q once, then a stage of keys (warp 0) and of values (warp 6) per
    // tile.  A load brings one unit of 16 rows; lane u issues unit u of its tile, with its own look-up
    // in the block table, so a tile's loads leave together.
    const bool is_v = warp == 6;
    if (!is_v && lane == 0) {
      mbar_expect_tx(&q_full, 16384);
      tma_load_2d(q_s, &map_q, &q_full, h * AT_HD, row0);
    }
    const int u = lane;
    const bool active = u < AT_BN / AT_UNIT;
    bool ok = true;
    // keys outside [key_lo, pos_last] are masked; their rows are read from the nearest unit of the
    // request that is there (finite values, weight zero)
    auto unit_row = [&](int it) -> int {
      if (!active || it >= n_it) return -1;
      int j = (tile_first + it) * AT_BN + u * AT_UNIT;
      j = max(min(j, pos_last), key_lo) / AT_UNIT * AT_UNIT;
      const int page = table[j / prm.page_size];
      if (page < 0 || page >= prm.n_pages) {
        *prm.status = NIB_STATUS_BAD_PAGE;
        return hk * prm.page_size;   // (page 0: in the pool)
      }
      return ((page * 2) * prm.n_kv_head + hk) * prm.page_size + j % prm.page_size;
    };
    // The two warps run loops of their own: the keys' warp is held back only by the scores (a stage's
    // keys are free as soon as the scores are made from them), the values' warp by the P V products,
    // so the keys that the scores three tiles ahead wait for leave early.
    uint8_t* dst_base = (is_v ? v_s : k_s) + u * 2048;
    const int row_off = is_v ? prm.n_kv_head * prm.page_size : 0;
    int row_next = unit_row(0);
    for (int it = 0; it < n_it; ++it) {
      const int st = it % AT_STAGES, round = it / AT_STAGES;
      const int row = row_next;
      row_next = unit_row(it + 1);   // the next tile's look-up travels while this tile's stage is waited for
      uint64_t* empty = is_v ? &v_empty[st] : &k_empty[st];
      uint64_t* full = is_v ? &v_full[st] : &k_full[st];
      if (round > 0) ok = warp_mbar_wait(empty, (round + 1) & 1, abort_flag, lane);
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(full, AT_KV_STAGE);
      __syncwarp();
      if (active) tma_load_2d(dst_base + st * AT_KV_STAGE, &map_kv, full, 0, row + row_off);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(AT_BM, AT_BN);
      const uint32_t idesc_o = umma_idesc(AT_BM, AT_HD) | (1u << 16);   // B (= V) is MN-major: keys down the rows
      const uint32_t o_tmem = tmem_base + O_COL;
      // scores of tile `it` into buffer it % AT_NBUF (free: P of tile it - AT_NBUF was made from it)
      auto issue_s = [&](int it) -> bool {
        const int st = it % AT_STAGES;
        if (!mbar_wait(&k_full[st], (it / AT_STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(q_s), kb = smem_u32(k_s + st * AT_KV_STAGE);
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k)   // 16 of the head's 64 values per instruction: 32 bytes along the row
          umma_bf16(tmem_base + (uint32_t)((it % AT_NBUF) * AT_BN), umma_desc(qa + k * 32), umma_desc(kb + k * 32),
                    idesc_s, k > 0);
        umma_commit(&s_full[it % AT_NBUF]);
        umma_commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(&q_full, 0, abort_flag);
      if (ok) ok = issue_s(0);
      for (int a = 1; ok && a < AT_NBUF && a < n_it; ++a) ok = issue_s(a);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % AT_STAGES, b = it % AT_NBUF;
        if (!mbar_wait(&v_full[st], (it / AT_STAGES) & 1, abort_flag)) break;
        if (!mbar_wait(&p_full[b], (it / AT_NBUF) & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t vb = smem_u32(v_s + st * AT_KV_STAGE);
        const uint32_t pa = smem_u32(p_s + b * P_BYTES);
#pragma unroll
        for (int k = 0; k < AT_BN / 16; ++k)   // 16 keys per instruction: P 32 bytes along its row, V 16 rows down
          umma_bf16(o_tmem, umma_desc(pa + (k >> 2) * 16384 + (k & 3) * 32), umma_desc(vb + k * 2048), idesc_o,
                    (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&o_full[b]);
        umma_commit(&v_empty[st]);
        if (it + AT_NBUF < n_it) ok = issue_s(it + AT_NBUF);
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax: a thread per row; warp w owns tensor-memory lanes 32 * (w % 4) .. +32
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int p = pos_first + r;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int wp0 = pos_first + quarter * 32, wp1 = wp0 + 31;   // positions of the warp's rows
    const float scale2 = prm.scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int b = it % AT_NBUF;
      ok = warp_mbar_wait(&s_full[b], (it / AT_NBUF) & 1, abort_flag, lane);
      if (!ok) break;
      tc_fence_after();
      const int j0 = (tile_first + it) * AT_BN;
      const bool edge = j0 + AT_BN - 1 > wp0 || (window > 0 && j0 < wp1 - window + 1);   // only these tiles need the mask
      float v[AT_BN];
#pragma unroll
      for (int c = 0; c < AT_BN / 32; ++c) tmem_ld32(lane_addr + (uint32_t)(b * AT_BN + c * 32), v + c * 32);
      if (edge) {
#pragma unroll
        for (int i = 0; i < AT_BN; ++i)
          if (!(j0 + i <= p && j0 + i >= lo)) v[i] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of 64 links
#pragma unroll
      for (int i = 0; i < AT_BN; i += 4) {
        mx4[0] = fmaxf(mx4[0], v[i]);
        mx4[1] = fmaxf(mx4[1], v[i + 1]);
        mx4[2] = fmaxf(mx4[2], v[i + 2]);
        mx4[3] = fmaxf(mx4[3], v[i + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= scale2;   // (scale2 > 0)
      // Raise the running maximum?  At the first tile it is set; later only when some row of the warp
      // exceeds its own by more than 2^AT_RAISE (or has had no key yet), and then O is scaled down.
      const bool raise = it == 0 || __any_sync(0xffffffffu, mx > m + AT_RAISE || (m == -INFINITY && mx > m));
      if (raise) {
        const float m_new = fmaxf(m, mx);
        if (it > 0) {
          const float corr = (m_new == -INFINITY) ? 1.0f : at_pow2(m - m_new);
          l *= corr;
          // O holds the tiles up to it - 1 once their MMAs are done
          ok = warp_mbar_wait(&o_full[(it - 1) % AT_NBUF], ((it - 1) / AT_NBUF) & 1, abort_flag, lane);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < AT_HD / 32; ++c) {
            float t[32];
            tmem_ld32(lane_addr + O_COL + (uint32_t)(c * 32), t);
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] *= corr;
            tmem_st32(lane_addr + O_COL + (uint32_t)(c * 32), t);
          }
        }
        m = m_new;
      }
      // a row with no key yet (all masked so far) keeps m = -inf; 2^(-inf - -inf) is avoided
      const float ms = (m == -INFINITY) ? 0.0f : m;
      // P of tile it - AT_NBUF (the last user of this buffer) has been read by its MMA
      if (it >= AT_NBUF) {
        ok = warp_mbar_wait(&o_full[b], ((it - AT_NBUF) / AT_NBUF) & 1, abort_flag, lane);
        if (!ok) break;
      }
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint8_t* blk0 = p_s + b * P_BYTES + r * 128;
#pragma unroll
      for (int g = 0; g < AT_BN / 8; ++g) {
        uint8_t* blk = blk0 + (g >> 3) * 16384;   // 64 keys (eight 16-byte pieces) a block
        float e8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e8[i] = at_pow2(fmaf(v[8 * g + i], scale2, -ms));   // 0 for a masked key
          sum4[i & 3] += e8[i];
        }
        *reinterpret_cast<uint4*>(blk + (((g & 7) ^ (r & 7)) * 16)) =
            make_uint4(pack_bf16(e8[0], e8[1]), pack_bf16(e8[2], e8[3]), pack_bf16(e8[4], e8[5]), pack_bf16(e8[6], e8[7]));
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMAs
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_full[b])) : "memory");
    }
    // the last MMA into O
    if (ok) ok = warp_mbar_wait(&o_full[(n_it - 1) % AT_NBUF], ((n_it - 1) / AT_NBUF) & 1, abort_flag, lane);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      bf16* dst = prm.out + (size_t)(row0 + r) * prm.ldo + h * AT_HD;
#pragma unroll 1
      for (int c = 0; c < AT_HD / 32; ++c) {
        float t[32];
        tmem_ld32(lane_addr + O_COL + (uint32_t)(c * 32), t);
        if (r < n_rows) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * g) = make_uint4(
                pack_bf16(t[8 * g] * inv, t[8 * g + 1] * inv), pack_bf16(t[8 * g + 2] * inv, t[8 * g + 3] * inv),
                pack_bf16(t[8 * g + 4] * inv, t[8 * g + 5] * inv), pack_bf16(t[8 * g + 6] * inv, t[8 * g + 7] * inv));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && abort_sh) *prm.status = NIB_STATUS_WAIT_TIMEOUT;
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace nib

using namespace nib;

// 1 if the tcgen05 prefill attention takes this shape (else the warp-level MMA kernel does).
extern "C" int nib_attention_prefill_tc_supported(int head_dim, int page_size) {
  return head_dim == AT_HD && page_size >= AT_UNIT && page_size % AT_UNIT == 0;
}

// tiles: n_tiles pairs (entry, first row within the entry), 128 rows each (the last of an entry may be
// shorter).  q [T, ldq] holds the queries of the step's T rows in its first n_head * 64 columns; cache
// is one layer [n_pages, 2, n_kv_head, page_size, 64]; out rows must be 16-byte aligned.
extern "C" int nib_attention_prefill_tc(const void* q, int ldq, int T, const void* cache, void* out, int ldo,
                                        const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                        const int* entry_start, const int* entry_pos0, int n_head, int n_kv_head,
                                        int head_dim, int page_size, int n_pages, float scale, int window,
                                        int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!nib_attention_prefill_tc_supported(head_dim, page_size)) return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_kv_head <= 0 || n_head % n_kv_head != 0 || !(scale > 0.0f) || T <= 0) return NIB_ERR_BAD_ARGUMENT;
  if ((ldq & 7) || ((uintptr_t)q & 15) || (ldo & 7) || ((uintptr_t)out & 15) || ((uintptr_t)cache & 15))
    return NIB_ERR_UNSUPPORTED_SIZE;
  if (n_tiles > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const long long kv_rows = (long long)n_pages * 2 * n_kv_head * page_size;
  if (kv_rows > 0x7fffffffll) return NIB_ERR_UNSUPPORTED_SIZE;
  CUtensorMap map_q, map_kv;
  if (!make_map(&map_q, q, false, T, n_head * AT_HD, ldq, AT_BM, AT_HD, true)) return NIB_ERR_DRIVER;
  if (!make_map(&map_kv, cache, false, (int)kv_rows, AT_HD, AT_HD, AT_UNIT, AT_HD, true)) return NIB_ERR_DRIVER;
  AtParams prm;
  prm.block_table = block_table; prm.max_blocks = max_blocks; prm.tiles = tiles;
  prm.entry_start = entry_start; prm.entry_pos0 = entry_pos0;
  prm.n_head = n_head; prm.n_kv_head = n_kv_head; prm.page_size = page_size; prm.n_pages = n_pages;
  prm.scale = scale; prm.window = window; prm.out = (bf16*)out; prm.ldo = ldo; prm.status = status;
  // 128 keys a tile, one block an SM: measured a little faster than 64 keys a tile and two blocks
  constexpr int BN = 128;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AtShape<BN>::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  launch_pdl(attention_prefill_tc_kernel<BN>, dim3(n_head, n_tiles), dim3(AT_THREADS), AtShape<BN>::SMEM, stream, map_q,
             map_kv, prm);
  NIB_LAUNCH_CHECK();
}

