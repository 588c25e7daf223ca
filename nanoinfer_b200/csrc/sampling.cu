// Greedy and temperature / top-k sampling on the device, one block per logits row.
//
// Semantics are the reference sampler's (crates/core/src/sampler.rs:4-78):
//   * temperature <= 0: argmax, ties to the lowest index;
//   * else scaled = logits / temperature; probabilities are the softmax over the FULL
//     vocabulary (maximum subtracted); the top_k most likely are kept (0 = all), highest
//     first; r = u * (sum of the kept probabilities); walk the kept tokens subtracting
//     each probability until r <= 0;
//   * u comes from a xorshift64* generator: u = (r >> 40) / 2^24.
// Here the generator's state, the temperature and top_k belong to the request: they live in
// per-slot arrays indexed by the row's state slot, so a request's draws do not depend on what
// else is in the batch.
//
// Instead of sorting, the walk is a radix select over order-preserving keys of the
// scaled logits, four passes of eight bits: first by count (which key is the k-th
// largest), then by probability mass (where the running sum reaches r).  Mass is kept
// in 32.32 fixed point so that the sums do not depend on the order of the additions.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_CHUNKS = 16;   // blocks that share a greedy row

__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
// exp(s - mx) in 32.32 fixed point; s <= mx so the value is at most 2^32.
__device__ __forceinline__ unsigned long long mass_of(float s, float mx) {
  return __float2ull_rz(expf(s - mx) * 4294967296.0f);
}

struct BestPair {
  float v;
  int i;
};
__device__ __forceinline__ BestPair better(BestPair a, BestPair b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// argmax of row[0..V) with ties to the lowest index; result valid in every thread.
__device__ int block_argmax(const float* __restrict__ row, int V, BestPair* scratch) {
  BestPair best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best.v) best = BestPair{v, i};  // indices rise within a thread: first maximum stays
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  BestPair r = (lane < n_warps) ? scratch[lane] : BestPair{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPair other{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = better(r, other);
  }
  return r.i == 0x7fffffff ? 0 : r.i;
}

__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int ld, int V,
                                                     int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  __shared__ BestPair scratch[32];
  const int r = blockIdx.x;
  const int best = block_argmax(logits + (size_t)r * ld, V, scratch);
  if (threadIdx.x == 0) out[r] = best;
}

struct SelectShared {
  unsigned long long hist[256];
  unsigned long long target;
  unsigned long long total;
  uint32_t digit;
  int count;
  int first;
};

// One radix select.  MASS = false: weights are 1 and `target` is a rank (1-based, from the
// top).  MASS = true: weights are probability masses; elements with key <= thresh are left
// out except that `tie_mass` is added for the key `thresh` itself, and the target is
// u24 * total >> 24 (at least 1), computed from the first histogram.
template <bool MASS>
__device__ void radix_select(const float* __restrict__ row, int V, float temperature, float mx,
                             bool use_thresh, uint32_t thresh, unsigned long long tie_mass,
                             unsigned long long target, uint32_t u24, SelectShared& sh,
                             uint32_t& key_out, unsigned long long& resid_out) {
  uint32_t prefix = 0, mask = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float s = row[i] / temperature;
      const uint32_t key = float_key(s);
      if ((key & mask) != prefix) continue;
      unsigned long long w = 1ull;
      if (MASS) {
        if (use_thresh && key <= thresh) continue;
        w = mass_of(s, mx);
      }
      atomicAdd(&sh.hist[(key >> shift) & 255u], w);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (MASS && use_thresh && (thresh & mask) == prefix) sh.hist[(thresh >> shift) & 255u] += tie_mass;
      unsigned long long tgt = target;
      if (MASS && shift == 24) {
        unsigned long long total = 0ull;
        for (int d = 0; d < 256; ++d) total += sh.hist[d];
        // (u24 * total) >> 24 without overflow: total < 2^49
        const unsigned long long hi = __umul64hi((unsigned long long)u24, total);
        const unsigned long long lo = (unsigned long long)u24 * total;
        tgt = (hi << 40) | (lo >> 24);
        if (tgt < 1ull) tgt = 1ull;
        sh.total = total;
      }
      unsigned long long cum = 0ull;
      int d = 255;
      for (; d > 0; --d) {
        if (cum + sh.hist[d] >= tgt) break;
        cum += sh.hist[d];
      }
      sh.digit = (uint32_t)d;
      sh.target = tgt - cum;
    }
    __syncthreads();
    prefix |= sh.digit << shift;
    mask |= 0xffu << shift;
    target = sh.target;
    __syncthreads();
  }
  key_out = prefix;
  resid_out = target;
}

// Grid (SAMPLE_CHUNKS, rows).  A greedy row is spread over the chunks: every block takes a slice of
// the vocabulary, folds (value, index) into one 64-bit word per row with atomicMax (the value's
// order-preserving key in the high half, ~index in the low half: the largest value wins, ties go
// to the lowest index), and the block that arrives last writes the token and clears the words.
// A sampled row is the work of block 0 of its row alone.  `scratch` holds 2 words per row
// (the folded maximum and the arrival count), zero between launches.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const int* __restrict__ row_slot,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              unsigned long long* __restrict__ rng_state, int* __restrict__ out,
              int* __restrict__ last_token, unsigned long long* __restrict__ scratch) {
  pdl_trigger();
  pdl_wait();
  __shared__ BestPair best_scratch[32];
  __shared__ float red[32];
  __shared__ SelectShared sh;
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * ld;
  const int slot = row_slot[r];
  const float temp = temperature[slot];
  if (!(temp > 0.0f)) {
    const int per = (V + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per, n = min(per, V - begin);
    if (n > 0) {
      const int best = begin + block_argmax(row + begin, n, best_scratch);
      if (threadIdx.x == 0) {
        const unsigned long long word =
            ((unsigned long long)float_key(row[best]) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)best);
        atomicMax(&scratch[2 * r], word);
      }
    }
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned long long arrived = atomicAdd(&scratch[2 * r + 1], 1ull);
      if (arrived == gridDim.x - 1) {
        __threadfence();
        const unsigned long long word = atomicExch(&scratch[2 * r], 0ull);
        scratch[2 * r + 1] = 0ull;
        const int tok = (int)(0xffffffffu - (uint32_t)(word & 0xffffffffull));
        out[r] = tok;
        if (last_token != nullptr) last_token[row_slot[r]] = tok;
      }
    }
    return;
  }
  if (blockIdx.x != 0) return;
  // one draw of xorshift64*, kept per request
  __shared__ uint32_t u24_sh;
  if (threadIdx.x == 0) {
    unsigned long long s = rng_state[slot];
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    rng_state[slot] = s;
    u24_sh = (uint32_t)((s * 0x2545F4914F6CDD1Dull) >> 40);
  }
  float mxl = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mxl = fmaxf(mxl, row[i] / temp);
  const float mx = block_max(mxl, red);  // also orders the write of u24_sh
  const uint32_t u24 = u24_sh;

  int k = top_k[slot];
  bool use_thresh = false;
  uint32_t thresh = 0;
  unsigned long long tie_keep = 0ull, tie_mass = 0ull;
  if (k > 0 && k < V) {
    radix_select<false>(row, V, temp, mx, false, 0u, 0ull, (unsigned long long)k, 0u, sh, thresh, tie_keep);
    use_thresh = true;
    tie_mass = tie_keep * mass_of(key_float(thresh), mx);
  }
  uint32_t key;
  unsigned long long resid;
  radix_select<true>(row, V, temp, mx, use_thresh, thresh, tie_mass, 0ull, u24, sh, key, resid);

  // the tokens that carry `key`, lowest index first; the walk stops at the n-th of them
  if (threadIdx.x == 0) {
    sh.count = 0;
    sh.first = 0x7fffffff;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (float_key(row[i] / temp) == key) {
      atomicAdd(&sh.count, 1);
      atomicMin(&sh.first, i);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long c = sh.count;
    if (use_thresh && key == thresh && (long long)tie_keep < c) c = (long long)tie_keep;
    const unsigned long long qk = mass_of(key_float(key), mx);
    long long n = qk > 0ull ? (long long)((resid + qk - 1ull) / qk) : 1;
    if (n < 1) n = 1;
    if (n > c) n = c;
    int tok = sh.first;
    if (n > 1) {
      long long seen = 0;
      for (int i = 0; i < V; ++i) {
        if (float_key(row[i] / temp) == key && ++seen == n) {
          tok = i;
          break;
        }
      }
    }
    tok = (tok == 0x7fffffff) ? 0 : tok;
    out[r] = tok;
    if (last_token != nullptr) last_token[row_slot[r]] = tok;
  }
}

}  // namespace nib

using namespace nib;

extern "C" int nib_argmax(const float* logits, int ld, int n_rows, int V, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  launch_pdl(argmax_kernel, dim3(n_rows), dim3(256), 0, stream, logits, ld, V, out);
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_sample(const float* logits, int ld, int n_rows, int V, const int* row_slot,
                          const float* temperature, const int* top_k, unsigned long long* rng_state,
                          int* out, int* last_token, unsigned long long* scratch, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_rows > 65535 || scratch == nullptr) return NIB_ERR_BAD_ARGUMENT;
  dim3 grid(SAMPLE_CHUNKS, n_rows);
  launch_pdl(sample_kernel, dim3(grid), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, row_slot, temperature, top_k, rng_state, out,
                                                     last_token, scratch);
  NIB_LAUNCH_CHECK();
}
