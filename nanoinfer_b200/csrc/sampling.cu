// Greedy and temperature / top-k sampling on the device: a greedy row is shared by sixteen blocks,
// a sampled row by the eight blocks of a cluster (or is one block's work when there are many).
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
// Instead of sorting, the walk is two selects over order-preserving keys of the scaled
// logits: first by count (which key is the k-th largest), then by probability mass (where
// the running sum reaches r).  A select sorts the row into bins that are linear in the
// distance from the maximum, picks the bin, and settles the exact key among that bin's few
// tokens with four passes of eight bits.  Mass is kept in 32.32 fixed point so that the
// sums do not depend on the order of the additions.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_CHUNKS = 16;   // blocks that share a greedy row
constexpr int SAMPLE_TEAM = 8;      // blocks (one cluster) that share a sampled row

// The blocks that work on one sampled row: this block alone (n = 1), or the n blocks of its cluster.
// Every block of a team passes the same sync() calls in the same order: none stands inside a
// branch that differs between the blocks of a team.
struct Team {
  int rank, n;
  __device__ __forceinline__ void sync() const {
    if (n > 1) {
      cluster_arrive();
      cluster_wait();
    } else {
      __syncthreads();
    }
  }
};

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

__global__ void __launch_bounds__(256) argmax_kernel(const float* logits, int ld, int V, int* out) {
  pdl_trigger();
  pdl_wait();
  __shared__ BestPair scratch[32];
  const int r = blockIdx.x;
  const int best = block_argmax(logits + (size_t)r * ld, V, scratch);
  if (threadIdx.x == 0) out[r] = best;
}

constexpr int SEL_BINS = 1024;        // coarse bins of the first pass
constexpr float SEL_SPAN = 24.0f;     // e^-24 * 2^32 < 1: a token that far below the maximum has no mass
constexpr int SEL_LIST = 2048;        // tokens of the chosen bin that are listed in shared memory

struct SelectShared {
  unsigned long long hist[256];
  uint32_t lo[SEL_BINS], hi[SEL_BINS];   // the coarse histogram, 64-bit sums in two halves
  uint32_t list_key[SEL_LIST];           // the chosen bin's tokens: their keys ...
  int list_idx[SEL_LIST];                // ... and indices (in no particular order)
  int n_list;                            // how many the bin has (the lists hold the first SEL_LIST)
  float peer_max[SAMPLE_TEAM];           // the maxima of the team's blocks
  uint32_t pub_thresh;                   // the first select's key, for the other blocks of the team
  unsigned long long target;
  unsigned long long total;
  uint32_t digit;
  int bin;
  int count;
  int first;
};

// The coarse bin of a scaled logit: bin 0 holds the maximum, the bins go down in steps of
// SEL_SPAN / (SEL_BINS - 1), the last bin holds everything further down (and NaNs).  Every step of
// the mapping is monotone, so all of a bin's tokens are larger than all of the next bin's.
__device__ __forceinline__ int coarse_bin(float s, float mx) {
  const float t = (mx - s) * ((float)(SEL_BINS - 1) / SEL_SPAN);
  return t < (float)(SEL_BINS - 1) ? (int)t : SEL_BINS - 1;
}

// One select.  MASS = false: weights are 1 and `target` is a rank (1-based, from the top).
// MASS = true: weights are probability masses; elements with key <= thresh are left out except that
// `tie_mass` is added for the key `thresh` itself, and the target is u24 * total >> 24 (at least 1).
//
// A radix select over the keys' bytes alone would start with the byte that holds the sign and most
// of the exponent, where logits crowd into a handful of values: fifty thousand atomic adds on a few
// shared words (64-bit ones are compare-and-swap loops) took most of a millisecond.  So the first
// pass sorts the tokens into SEL_BINS bins that are linear in the distance from the maximum, where
// they spread out, with native 32-bit atomic adds (a 64-bit sum is kept as two halves with a carry;
// integer sums do not depend on the order of the additions).  A warp finds the bin in which the
// target falls; one more pass lists that bin's tokens (a few dozen to a few hundred) in shared
// memory, and the four byte passes settle the exact key among the listed ones.  A bin with more
// than SEL_LIST tokens (logits that are nearly all alike) is not listed: the byte passes then walk
// the whole row as the first pass does.
template <bool MASS>
__device__ void radix_select(const float* __restrict__ row, int V, float temperature, float mx,
                             bool use_thresh, uint32_t thresh, unsigned long long tie_mass,
                             unsigned long long target, uint32_t u24, SelectShared& sh, const Team team,
                             uint32_t& key_out, unsigned long long& resid_out) {
  // With a team, every block takes a slice of the row for the passes over all tokens; the first
  // block adds the histograms up, picks the bin, owns the list (the others append to it through
  // distributed shared memory) and does the byte passes alone.
  const int per = (V + team.n - 1) / team.n;
  const int v0 = min(V, team.rank * per), v1 = min(V, v0 + per);
  const int thresh_bin = (MASS && use_thresh) ? coarse_bin(key_float(thresh), mx) : -1;
  for (int i = threadIdx.x; i < SEL_BINS; i += blockDim.x) sh.lo[i] = sh.hi[i] = 0u;
  __syncthreads();
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const float s = row[i] / temperature;
    if (MASS) {
      if (use_thresh && float_key(s) <= thresh) continue;
      const unsigned long long w = mass_of(s, mx);
      const uint32_t wl = (uint32_t)w, wh = (uint32_t)(w >> 32);
      const int b = coarse_bin(s, mx);
      if (wl) {
        const uint32_t old = atomicAdd(&sh.lo[b], wl);
        if (old + wl < old) atomicAdd(&sh.hi[b], 1u);
      }
      if (wh) atomicAdd(&sh.hi[b], wh);
    } else {
      atomicAdd(&sh.lo[coarse_bin(s, mx)], 1u);
    }
  }
  team.sync();   // every block's histogram is complete
  if (team.rank == 0) {
    if (team.n > 1) {
      for (int b = threadIdx.x; b < SEL_BINS; b += blockDim.x) {
        unsigned long long v = ((unsigned long long)sh.hi[b] << 32) | sh.lo[b];
        for (int r = 1; r < team.n; ++r)
          v += ((unsigned long long)cluster_load(cluster_addr(&sh.hi[b], r)) << 32) | cluster_load(cluster_addr(&sh.lo[b], r));
        sh.lo[b] = (uint32_t)v;
        sh.hi[b] = (uint32_t)(v >> 32);
      }
      __syncthreads();
    }
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      constexpr int PER = SEL_BINS / 32;
      if (MASS && use_thresh && thresh_bin / PER == lane) {   // the kept ties of the threshold key
        const unsigned long long v = (((unsigned long long)sh.hi[thresh_bin] << 32) | sh.lo[thresh_bin]) + tie_mass;
        sh.lo[thresh_bin] = (uint32_t)v;
        sh.hi[thresh_bin] = (uint32_t)(v >> 32);
      }
      unsigned long long mine = 0ull;
      for (int b = lane * PER; b < (lane + 1) * PER; ++b) mine += ((unsigned long long)sh.hi[b] << 32) | sh.lo[b];
      unsigned long long incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const unsigned long long total = __shfl_sync(0xffffffffu, incl, 31);
      unsigned long long tgt = target;
      if (MASS) {
        // (u24 * total) >> 24 without overflow: total < 2^49
        const unsigned long long hi = __umul64hi((unsigned long long)u24, total);
        const unsigned long long lo = (unsigned long long)u24 * total;
        tgt = (hi << 40) | (lo >> 24);
        if (tgt < 1ull) tgt = 1ull;
      }
      const uint32_t reached = __ballot_sync(0xffffffffu, incl >= tgt);
      const int owner = reached ? __ffs(reached) - 1 : 31;
      if (lane == owner) {
        unsigned long long cum = incl - mine;
        int b = lane * PER;
        for (; b < (lane + 1) * PER - 1; ++b) {
          const unsigned long long h = ((unsigned long long)sh.hi[b] << 32) | sh.lo[b];
          if (cum + h >= tgt) break;
          cum += h;
        }
        sh.bin = b;
        sh.target = tgt - cum;
        sh.total = total;
        sh.n_list = 0;
      }
    }
  }
  team.sync();   // the bin is chosen (and the first block has read the others' histograms)
  const int bin = team.rank == 0 ? sh.bin : (int)cluster_load(cluster_addr(&sh.bin, 0));
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const float s = row[i] / temperature;
    if (coarse_bin(s, mx) != bin) continue;
    const uint32_t key = float_key(s);
    if (MASS && use_thresh && key <= thresh) continue;
    if (team.rank == 0) {
      const int at = atomicAdd(&sh.n_list, 1);
      if (at < SEL_LIST) {
        sh.list_key[at] = key;
        sh.list_idx[at] = i;
      }
    } else {
      const int at = (int)cluster_atomic_add(cluster_addr(&sh.n_list, 0), 1u);
      if (at < SEL_LIST) {
        cluster_store(cluster_addr(&sh.list_key[at], 0), key);
        cluster_store(cluster_addr(&sh.list_idx[at], 0), (uint32_t)i);
      }
    }
  }
  team.sync();   // the list is complete
  if (team.rank != 0) return;   // (the caller's next sync() is the next one for every block)
  target = sh.target;
  const int n_list = sh.n_list;
  const bool listed = n_list <= SEL_LIST;

  uint32_t prefix = 0, mask = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0ull;
    __syncthreads();
    if (listed) {
      for (int j = threadIdx.x; j < n_list; j += blockDim.x) {
        const uint32_t key = sh.list_key[j];
        if ((key & mask) != prefix) continue;
        atomicAdd(&sh.hist[(key >> shift) & 255u], MASS ? mass_of(key_float(key), mx) : 1ull);
      }
    } else {
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float s = row[i] / temperature;
        if (coarse_bin(s, mx) != bin) continue;
        const uint32_t key = float_key(s);
        if ((key & mask) != prefix) continue;
        unsigned long long w = 1ull;
        if (MASS) {
          if (use_thresh && key <= thresh) continue;
          w = mass_of(s, mx);
        }
        atomicAdd(&sh.hist[(key >> shift) & 255u], w);
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // the digit in which the target falls, from the top: a lane per eight digits, a scan over the
      // lanes, then the owning lane walks its eight (one thread walking all 256 cost 5 us a pass)
      const int lane = threadIdx.x;
      const int top = 255 - 8 * lane;
      if (MASS && use_thresh && thresh_bin == bin && (thresh & mask) == prefix &&
          (255 - (int)((thresh >> shift) & 255u)) / 8 == lane)
        sh.hist[(thresh >> shift) & 255u] += tie_mass;
      unsigned long long mine = 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += sh.hist[top - j];
      unsigned long long incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const uint32_t reached = __ballot_sync(0xffffffffu, incl >= target);
      const int owner = reached ? __ffs(reached) - 1 : 31;
      if (lane == owner) {
        unsigned long long cum = incl - mine;
        int d = top;
        for (; d > top - 7; --d) {
          if (cum + sh.hist[d] >= target) break;
          cum += sh.hist[d];
        }
        sh.digit = (uint32_t)d;
        sh.target = target - cum;
      }
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
// A sampled row is the work of the first `team_size` blocks of its row: block 0 alone, or (launched
// as clusters of SAMPLE_TEAM blocks) one cluster, whose blocks share the passes over all tokens.
// `scratch` holds 2 words per row (the folded maximum and the arrival count), zero between launches.
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_kernel(const float* logits, int ld, int V, const int* __restrict__ row_slot,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              unsigned long long* rng_state, int* out,
              int* last_token, unsigned long long* scratch, int team_size) {
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
  // ---- a sampled row: the first `team` blocks of the row's grid line (one cluster, or block 0 alone)
  if ((int)blockIdx.x >= team_size) return;
  const Team team{team_size > 1 ? cluster_rank() : 0, team_size};
  team.sync();   // every block of the team runs: its shared memory may be written from now on
  // one draw of xorshift64*, kept per request
  __shared__ uint32_t u24_sh;
  if (team.rank == 0 && threadIdx.x == 0) {
    unsigned long long s = rng_state[slot];
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    rng_state[slot] = s;
    u24_sh = (uint32_t)((s * 0x2545F4914F6CDD1Dull) >> 40);
  }
  float mxl = -INFINITY;
  {
    const int per = (V + team.n - 1) / team.n;
    const int v0 = min(V, team.rank * per), v1 = min(V, v0 + per);
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) mxl = fmaxf(mxl, row[i] / temp);
  }
  float mx = block_max(mxl, red);  // also orders the write of u24_sh
  if (team.n > 1) {   // every block tells every block its maximum
    if ((int)threadIdx.x < team.n)
      cluster_store(cluster_addr(&sh.peer_max[team.rank], threadIdx.x), __float_as_uint(mx));
    team.sync();
    for (int r = 0; r < team.n; ++r) mx = fmaxf(mx, sh.peer_max[r]);
  }
  const uint32_t u24 = u24_sh;

  int k = top_k[slot];
  bool use_thresh = false;
  uint32_t thresh = 0;
  unsigned long long tie_keep = 0ull, tie_mass = 0ull;
  if (k > 0 && k < V) {   // (the same for every block of the team)
    radix_select<false>(row, V, temp, mx, false, 0u, 0ull, (unsigned long long)k, 0u, sh, team, thresh, tie_keep);
    use_thresh = true;
    if (team.n > 1) {   // the first block found the k-th key: the others need it for their slices
      if (team.rank == 0 && threadIdx.x == 0) sh.pub_thresh = thresh;
      team.sync();
      if (team.rank != 0) thresh = cluster_load(cluster_addr(&sh.pub_thresh, 0));
    }
    tie_mass = tie_keep * mass_of(key_float(thresh), mx);   // (used by the first block only)
  }
  uint32_t key;
  unsigned long long resid;
  radix_select<true>(row, V, temp, mx, use_thresh, thresh, tie_mass, 0ull, u24, sh, team, key, resid);
  if (team.rank != 0) return;   // (after the last sync(): nothing reads this block's shared memory any more)

  // the tokens that carry `key`, lowest index first; the walk stops at the n-th of them
  if (threadIdx.x == 0) {
    sh.count = 0;
    sh.first = 0x7fffffff;
  }
  __syncthreads();
  // (the last select's list holds every token of the chosen key's bin, unless it was too long;
  // a threshold key's own tokens are not in it: they are left out of the masses and re-enter as ties)
  const bool from_list = sh.n_list <= SEL_LIST && !(use_thresh && key == thresh);
  if (from_list) {
    for (int j = threadIdx.x; j < sh.n_list; j += blockDim.x) {
      if (sh.list_key[j] == key) {
        atomicAdd(&sh.count, 1);
        atomicMin(&sh.first, sh.list_idx[j]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      if (float_key(row[i] / temp) == key) {
        atomicAdd(&sh.count, 1);
        atomicMin(&sh.first, i);
      }
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
    if (n > 1 && from_list) {        // the n-th lowest index among the listed tokens of the key
      for (long long seen = 1; seen < n; ++seen) {
        int next = 0x7fffffff;
        for (int j = 0; j < sh.n_list; ++j)
          if (sh.list_key[j] == key && sh.list_idx[j] > tok && sh.list_idx[j] < next) next = sh.list_idx[j];
        tok = next;
      }
    } else if (n > 1) {
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
                          int* out, int* last_token, unsigned long long* scratch, int teams,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_rows > 65535 || scratch == nullptr) return NIB_ERR_BAD_ARGUMENT;
  // teams != 0: some rows may be sampled, and the launch is made of clusters of SAMPLE_TEAM blocks
  // (a greedy row does not care); a launch of greedy rows only needs no clusters
  static_assert(SAMPLE_CHUNKS % SAMPLE_TEAM == 0, "a row's grid line is whole clusters");
  // (the largest of 8, 4 and 2 blocks with which all rows' teams are on the device at once, as the runtime
  // counts clusters of that size: a team too many waits for a wave to end; beyond that a row is one block's work)
  int team = 1;
  if (teams) {
    static int room[SAMPLE_TEAM + 1] = {};     // clusters of t blocks that the device holds at once (0: not asked yet)
    for (int t = SAMPLE_TEAM; t > 1; t /= 2) {
      if (room[t] == 0) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(t, 148);
        q.blockDim = dim3(SAMPLE_THREADS);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = t;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        q.attrs = attr;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, sample_kernel, &q) != cudaSuccess || n < 1) n = -1;
        room[t] = n;
      }
      if (n_rows <= room[t]) { team = t; break; }
    }
  }
  // Blocks per row: as many as keep the grid within one wave (a block of 1024 threads has an SM to
  // itself), at most SAMPLE_CHUNKS, and whole clusters where there are teams.
  int chunks = SAMPLE_CHUNKS;
  while (chunks > team && n_rows * chunks > 148) chunks /= 2;
  dim3 grid(chunks, n_rows);
  launch_pdl_cluster(sample_kernel, dim3(grid), dim3(SAMPLE_THREADS), 0, stream, team, logits, ld, V, row_slot,
                     temperature, top_k, rng_state, out, last_token, scratch, team);
  NIB_LAUNCH_CHECK();
}
