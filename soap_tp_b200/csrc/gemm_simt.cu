// Plain fp32 FMA GEMM on CUDA cores with arbitrary operand strides (see gemm.h).  32x32 output tile
// per CTA, 16-deep k slices staged through shared memory, 2x2 outputs per thread.
#include <stdexcept>
#include <string>

#include "gemm.h"

namespace soapb200 {
namespace {

constexpr int kTile = 32;
constexpr int kDepth = 16;

__global__ void __launch_bounds__(256) gemm_simt_kernel(const float* __restrict__ A, int64_t a_sk, int64_t a_sm,
                                                        const float* __restrict__ B, int64_t b_sk, int64_t b_sn,
                                                        float* __restrict__ C, int64_t c_sm, int64_t c_sn, int M, int N,
                                                        int K, float alpha, float beta) {
  __shared__ float As[kDepth][kTile + 1];
  __shared__ float Bs[kDepth][kTile + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.x * kTile, n0 = blockIdx.y * kTile;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += kDepth) {
    for (int i = threadIdx.x; i < kDepth * kTile; i += 256) {
      const int kk = i / kTile, mm = i % kTile;
      const int k = k0 + kk;
      As[kk][mm] = (k < K && m0 + mm < M) ? A[k * a_sk + (m0 + mm) * a_sm] : 0.f;
      Bs[kk][mm] = (k < K && n0 + mm < N) ? B[k * b_sk + (n0 + mm) * b_sn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kDepth; ++kk) {
      const float a0 = As[kk][tx], a1 = As[kk][tx + 16];
      const float b0 = Bs[kk][ty], b1 = Bs[kk][ty + 16];
      acc[0][0] = fmaf(a0, b0, acc[0][0]);
      acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]);
      acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = m0 + tx + 16 * i, n = n0 + ty + 16 * j;
      if (m < M && n < N) {
        float* dst = C + m * c_sm + n * c_sn;
        float v = alpha * acc[i][j];
        if (beta != 0.f) v = fmaf(beta, *dst, v);
        *dst = v;
      }
    }
}

}  // namespace

void gemm_simt(const float* A, int64_t a_sk, int64_t a_sm, const float* B, int64_t b_sk, int64_t b_sn, float* C,
               int64_t c_sm, int64_t c_sn, int M, int N, int K, float alpha, float beta, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return;
  dim3 grid((M + kTile - 1) / kTile, (N + kTile - 1) / kTile);
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(A, a_sk, a_sm, B, b_sk, b_sn, C, c_sm, c_sn, M, N, K, alpha, beta);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("gemm_simt launch: ") + cudaGetErrorString(err));
}

}  // namespace soapb200
