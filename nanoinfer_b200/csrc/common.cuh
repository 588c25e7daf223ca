// Shared device helpers for the sm_100a kernels: storage types, conversions and
// warp/block reductions.  All arithmetic that decides a result's accuracy
// (statistics, softmax, accumulators, the residual sum) is done in 32-bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nib {

using bf16 = __nv_bfloat16;

// dtype codes of the C interface
enum : int { DT_F32 = 0, DT_BF16 = 1 };

// activation codes of the linear epilogues
enum : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// tanh form: 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3))); erf form: 0.5 u (1 + erf(u / sqrt 2)).
// tanhf and erff are the accurate library functions, never the approximate intrinsics.
__device__ __forceinline__ float gelu_tanh(float u) {
  const float k = 0.7978845608028654f;
  return 0.5f * u * (1.0f + tanhf(k * (u + 0.044715f * u * u * u)));
}
__device__ __forceinline__ float gelu_erf(float u) {
  return 0.5f * u * (1.0f + erff(u * 0.7071067811865476f));
}
__device__ __forceinline__ float apply_act(float u, int act) {
  if (act == ACT_GELU_TANH) return gelu_tanh(u);
  if (act == ACT_GELU_ERF) return gelu_erf(u);
  return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  The result
// is the same in every thread, and the order of the additions is fixed.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < n_warps) ? scratch[lane] : 0.0f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < n_warps) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

// Where token `pos` of a request lies in a paged cache layer laid out as
// [page][K|V][kv_head][slot in page][head_dim].
__device__ __forceinline__ size_t kv_offset(int page, int kv, int head, int slot, int n_kv_head,
                                            int page_size, int head_dim) {
  return ((((size_t)page * 2 + kv) * n_kv_head + head) * page_size + slot) * (size_t)head_dim;
}

// Programmatic dependent launch.  Every kernel of the library starts with pdl_trigger() (the next
// kernel in the stream may be scheduled and run its prologue while this one works) and calls
// pdl_wait() before its first access to global memory (which returns once the kernel before it has
// finished and its writes are visible).  A step is a chain of a hundred short kernels, and this
// hides each one's launch latency behind its predecessor.
//
// A rule that follows: a pointer to anything that a kernel of the same step writes (activations, the
// residual stream, queries, the cache, logits) is NEVER declared `const T* __restrict__`.  The compiler
// treats loads through such a pointer as invariant for the kernel's lifetime (ld.global.nc) and is
// free to move them above pdl_wait(), asm memory clobber or not; it did so in a kernel that asked for
// its weights before the wait, and read the step's rows there too, before they were written.  Only
// what no kernel of the step writes (weights, biases, norm parameters, the step's tables, which the
// host copied in before the step) may be read through a const __restrict__ pointer.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- thread-block clusters: rank, barrier, and a store into another block's shared memory
__device__ __forceinline__ int cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return (int)r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `local` in the shared memory of block `rank` of the cluster, and 32-bit accesses there
__device__ __forceinline__ uint32_t cluster_addr(const void* local, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ uint32_t cluster_load(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_store(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cluster_atomic_add(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}
// stores v at the place of `local` in the shared memory of block `rank` of the cluster
__device__ __forceinline__ void store_to_rank(float* local, int rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// 16 bytes from global to shared memory without passing through registers: many can be in flight
// per thread.  `valid` false reads nothing and fills the 16 bytes with zeros.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Launch with the programmatic-serialization attribute set.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a grid whose x dimension is cut into clusters of `cluster_x` blocks.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster_x > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace nib

#define NIB_LAUNCH_CHECK() return (int)cudaGetLastError()
