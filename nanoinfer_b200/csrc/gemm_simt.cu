// out = act(a . w^T + bias) on the CUDA cores, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (FFMA only: no tensor cores,
// hence no reduced-precision matrix mode) and the fallback of the bfloat16 path
// for shapes the tensor-core kernel refuses.  The weight is [N, K] ("out, in"),
// the layout the reference transposes to at load (crates/core/src/weights.rs:1-9),
// and the product is the reference's x . W^T + b (crates/core/src/kernels/reference.rs:26-37).
// Each output element is a single accumulator that adds its K products in index
// order, whatever the other rows of the batch are.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4 x 4 outputs each

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const InT* __restrict__ a, int lda, const InT* __restrict__ w, int ldw,
                   const float* __restrict__ bias, OutT* __restrict__ out, int ldo, int M, int N,
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

template <typename InT, typename OutT>
static int launch(const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                  int ldo, int M, int N, int K, int act, int residual, cudaStream_t stream) {
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
