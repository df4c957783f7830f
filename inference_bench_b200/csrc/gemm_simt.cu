// out[t][n] = sum_k x[t][k] * w[n][k] in float32 FMA arithmetic, for any T, N, K.
//
// This is the matrix product of the true 32-bit path (float32 inputs; no tensor-core mode of
// reduced precision), and with bfloat16 inputs it is the plain reference of the tcgen05 kernel.
// Every output element is one sequential chain of FMAs over k = 0..K-1, so a row's result does
// not depend on which other rows share the launch. The reference's equivalent is its 64x64x16
// float32 tile (crates/kir/src/cuda/prelude.cu:213-276).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename X, typename W>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const X* __restrict__ x, const W* __restrict__ w, float* __restrict__ out, int T,
                                                        int N, int K) {
  __shared__ float xs[BK][BM + 1];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  __shared__ float ws[BK][BN + 1];
  const int t0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;  // thread's 4x4 micro tile: rows ty*4.., cols tx*4..
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread.
#pragma unroll
    for (int e = 0; e < 4; e++) {
      int idx = tid + e * 256;
      int r = idx / BK, kk = idx % BK;
      int k = k0 + kk;
      int t = t0 + r, n = n0 + r;
      xs[kk][r] = (t < T && k < K) ? ib::to_f32<X>(x[(size_t)t * K + k]) : 0.f;
      ws[kk][r] = (n < N && k < K) ? ib::to_f32<W>(w[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    int t = t0 + ty * TM + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int n = n0 + tx * TN + j;
      if (n < N) out[(size_t)t * N + n] = acc[i][j];
    }
  }
}

}  // namespace

extern "C" int ib_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, float* out, int T, int N, int K, cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  IB_CHECK_ARG(T > 0 && N > 0 && K > 0, "gemm_simt: bad sizes T=%d N=%d K=%d", T, N, K);
  dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM);
  IB_CHECK_ARG(grid.y <= 65535, "gemm_simt: T=%d rows exceed the grid limit", T);
  if (x_dtype == IB_F32 && w_dtype == IB_F32)
    ib::launch(gemm_simt_kernel<float, float>, grid, 256, 0, stream, (const float*)x, (const float*)w, out, T, N, K);
  else if (x_dtype == IB_BF16 && w_dtype == IB_BF16)
    ib::launch(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, T, N, K);
  else if (x_dtype == IB_F32 && w_dtype == IB_BF16)
    ib::launch(gemm_simt_kernel<float, __nv_bfloat16>, grid, 256, 0, stream, (const float*)x, (const __nv_bfloat16*)w, out, T, N, K);
  else
    return ib_set_error("gemm_simt: unsupported dtypes x=%d w=%d", x_dtype, w_dtype);
  IB_CHECK_LAUNCH("gemm_simt");
  return 0;
}
