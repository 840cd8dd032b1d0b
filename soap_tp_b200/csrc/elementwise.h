// Host-side interface of the memory-bound kernels (elementwise.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace soapb200 {

// m <- b1 m + (1-b1) g;  v <- b2 v + (1-b2) g^2;  u = (m*inv_bc1) / (sqrt(v)*inv_sqrt_bc2 + eps).
// All four matrices are rows x cols, column-major, with their own pitches.
void adam_update(const float* g, int64_t ldg, float* m, int64_t ldm, float* v, int64_t ldv, float* u, int64_t ldu,
                 int rows, int cols, float beta1, float beta2, float eps, float inv_bc1, float inv_sqrt_bc2,
                 cudaStream_t stream);

// hi/lo planes of out(i, j) = scale * src[i*s_i + j*s_j]; planes are column-major with pitch ldo.  With `hl` (the
// interleaved bf16 plane of gemm.h, pitch ld16 elements) the low part goes there and `lo` is not written.
void split_planes(const float* src, int64_t s_i, int64_t s_j, float* hi, float* lo, int64_t ldo, int rows, int cols,
                  float scale, int nearest, cudaStream_t stream, uint16_t* hl = nullptr, int64_t ld16 = 0);

// out[j] = sum_i a[i, j] * b[i, j] for column-major a, b (deterministic tree reduction per column).
void column_dot(const float* a, int64_t lda, const float* b, int64_t ldb, float* out, int rows, int cols,
                cudaStream_t stream);

// order = stable descending argsort of estimates[j] = sum_{r < parts} table[r + j * ld], j < n <= kOrderMaxLength
// (one CTA, shared-memory bitonic sort; NaN estimates sort last).
constexpr int kOrderMaxLength = 16384;
void order_by_estimate(const float* table, int64_t ld, int parts, int n, int64_t* order, cudaStream_t stream);

// dst(i, j) = src(row_map[i], col_map[j]); a null map is the identity.
void gather2d(const float* src, int64_t s_i, int64_t s_j, float* dst, int64_t d_i, int64_t d_j, const int64_t* row_map,
              const int64_t* col_map, int rows, int cols, cudaStream_t stream);

}  // namespace soapb200
