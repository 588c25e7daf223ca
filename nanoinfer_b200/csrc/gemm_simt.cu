// out = act(a . w^T + bias) on the CUDA cores, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (FFMA only: no tensor cores,
// hence no reduced-precision matrix mode) and the fallback of the bfloat16 path
// for shapes the tensor-core kernel refuses.  The weight is [N, K] ("out, in"),
// the layout the reference transposes to at load (crates/core/src/weights.rs:1-9),
// and the product is the reference's x . W^T + b (crates/core/src/kernels/reference.rs:26-37).
// Each output element is a single accumulator that adds its K products in index
// order, whatever the other rows of the batch are.
#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4 x 4 outputs each

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const InT* a, int lda, const InT* __restrict__ w, int ldw,
                   const float* __restrict__ bias, OutT* out, int ldo, int M, int N,
                   int K, int act, int residual) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // tx -> columns, ty -> rows
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  // each thread stages 4 elements of each tile: row = tid / 4, k = (tid % 4) * 4 .. +4
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + i][lr] = (am < M && k < K) ? to_float(a[(size_t)am * lda + k]) : 0.0f;
      Ws[lk + i][lr] = (wn < N && k < K) ? to_float(w[(size_t)wn * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = apply_act(v, act);
      OutT* o = out + (size_t)m * ldo + n;
      if (residual) v += to_float(*o);
      *o = from_float<OutT>(v);
    }
  }
}

// The same product for steps of at most 16 rows.  The tiled kernel above leaves 63 of its 64 rows
// idle on a single decoded token and takes 48 dependent rounds of loads for K = 768.  Here a block owns
// 64 features and every thread one feature for ROWS / 4 of the step's rows; K comes in chunks of 64
// that are asked for two chunks ahead (registers), so that the chain is half as many rounds and each
// overlaps the one before.  Every output is still ONE accumulator that adds its K products in index
// order with the same fused multiply-adds: the bits are those of the tiled kernel, whatever the batch.
constexpr int RB_N = 64, RB_K = 64;

// (`a` and `out` carry no __restrict__: see pdl_wait in common.cuh.  With it, the compiler read the
// step's rows beside the weights, above the wait, before the kernel that writes them had finished.)
template <typename InT, typename OutT, int ROWS>
__global__ void __launch_bounds__(256)
linear_simt_rows_kernel(const InT* a, int lda, const InT* __restrict__ w, int ldw,
                        const float* __restrict__ bias, OutT* out, int ldo, int M, int N, int K,
                        int act, int residual) {
  constexpr int RPT = ROWS / 4;                      // rows per thread
  constexpr int WPT = RB_N * RB_K / 256;             // weight values a thread stages per chunk: 16
  constexpr int APT = (ROWS * RB_K + 255) / 256;     // values of the step's rows per thread and chunk
  pdl_trigger();
  __shared__ float Ws[2][RB_N][RB_K + 1];
  __shared__ float As[2][ROWS][RB_K];
  const int tid = threadIdx.x, n0 = blockIdx.x * RB_N;
  const int f = tid % RB_N, rg = tid / RB_N;
  const int lk = tid % RB_K, lr = tid / RB_K;        // staging: column of the chunk, first of the rows (step 4)
  float wreg[2][WPT], areg[2][APT];
  // asks for chunk c (columns c * 64 ...) into the register set `s`: weights do not depend on the kernel
  // ahead, the step's rows do
  auto ask_w = [&](int c, int s) {
#pragma unroll
    for (int j = 0; j < WPT; ++j) {
      const int n = n0 + lr + 4 * j, k = c * RB_K + lk;
      wreg[s][j] = (n < N && k < K) ? to_float(w[(size_t)n * ldw + k]) : 0.0f;
    }
  };
  auto ask_a = [&](int c, int s) {
#pragma unroll
    for (int j = 0; j < APT; ++j) {
      const int m = lr + 4 * j, k = c * RB_K + lk;
      areg[s][j] = (m < M && m < ROWS && k < K) ? to_float(a[(size_t)m * lda + k]) : 0.0f;
    }
  };
  const int n_chunks = (K + RB_K - 1) / RB_K;
  ask_w(0, 0);
  if (n_chunks > 1) ask_w(1, 1);
  pdl_wait();
  ask_a(0, 0);
  if (n_chunks > 1) ask_a(1, 1);
  float acc[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) acc[i] = 0.0f;
  // one chunk: the registers of set S go to buffer S, the chunk after next is asked for into them, and
  // the chunk's 64 products are added (S is a constant of the code, so that the sets stay in registers)
  auto chunk = [&](int c, auto S) {
    constexpr int s = decltype(S)::value;
#pragma unroll
    for (int j = 0; j < WPT; ++j) Ws[s][lr + 4 * j][lk] = wreg[s][j];
#pragma unroll
    for (int j = 0; j < APT; ++j) As[s][lr + 4 * j][lk] = areg[s][j];
    if (c + 2 < n_chunks) {
      ask_w(c + 2, s);
      ask_a(c + 2, s);
    }
    __syncthreads();          // (two buffers by turns: a buffer is written again two chunks later, a barrier between)
#pragma unroll 16
    for (int k = 0; k < RB_K; ++k) {
      const float wv = Ws[s][f][k];
#pragma unroll
      for (int i = 0; i < RPT; ++i) acc[i] = fmaf(As[s][rg * RPT + i][k], wv, acc[i]);
    }
  };
  for (int c = 0; c < n_chunks; c += 2) {
    chunk(c, std::integral_constant<int, 0>());
    if (c + 1 < n_chunks) chunk(c + 1, std::integral_constant<int, 1>());
  }
  const int n = n0 + f;
  if (n >= N) return;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int m = rg * RPT + i;
    if (m >= M) continue;
    float v = acc[i];
    if (bias) v += bias[n];
    v = apply_act(v, act);
    OutT* o = out + (size_t)m * ldo + n;
    if (residual) v += to_float(*o);
    *o = from_float<OutT>(v);
  }
}

template <typename InT, typename OutT>
static int launch(const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                  int ldo, int M, int N, int K, int act, int residual, cudaStream_t stream) {
  if (M <= 16) {
    const dim3 rgrid((N + RB_N - 1) / RB_N);
    if (M <= 8)
      launch_pdl(linear_simt_rows_kernel<InT, OutT, 8>, rgrid, dim3(256), 0, stream, (const InT*)a, lda, (const InT*)w,
                 ldw, bias, (OutT*)out, ldo, M, N, K, act, residual);
    else
      launch_pdl(linear_simt_rows_kernel<InT, OutT, 16>, rgrid, dim3(256), 0, stream, (const InT*)a, lda, (const InT*)w,
                 ldw, bias, (OutT*)out, ldo, M, N, K, act, residual);
    NIB_LAUNCH_CHECK();
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  launch_pdl(linear_simt_kernel<InT, OutT>, dim3(grid), dim3(256), 0, stream, (const InT*)a, lda, (const InT*)w, ldw, bias,
                                                          (OutT*)out, ldo, M, N, K, act, residual);
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

extern "C" int nib_linear_simt(int in_dtype, int out_dtype, const void* a, int lda, const void* w,
                               int ldw, const float* bias, void* out, int ldo, int M, int N, int K,
                               int act, int residual, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return NIB_ERR_BAD_ARGUMENT;
  if (residual && out_dtype != DT_F32) return NIB_ERR_BAD_ARGUMENT;  // the residual stream is 32-bit
  if ((M + BM - 1) / BM > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (in_dtype == DT_F32 && out_dtype == DT_F32)
    return launch<float, float>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
    return launch<bf16, bf16>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_F32)
    return launch<bf16, float>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, stream);
  return NIB_ERR_BAD_ARGUMENT;
}
