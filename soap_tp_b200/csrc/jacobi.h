// Host-side interface of the block-Jacobi eigensolver's small-problem kernel (jacobi.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace soapb200 {

// For every batch item b, the 128 x 128 diagonal block G_b of a symmetric matrix held as operand planes
// (entry (i, j) of block b at planes[(128 b + i) * lds + 128 b + j]) is diagonalised by cyclic two-sided
// Jacobi in shared memory, G_b = U_b diag U_b^T.  U_b is written as operand planes: element (k, n') at
// [k + (128 b + n') * ldu].  *offdiag receives (atomic max over all items, as float bits) the largest
// |G_ij| / scale, i != j, found BEFORE rotating: the convergence measure of the outer sweep.  Rotations
// are skipped for |G_pq| <= tolerance * scale.
void jacobi_small(const float* s_hi, const float* s_lo, int64_t lds, int batches, float* u_hi, float* u_lo, int64_t ldu,
                  float* offdiag, float scale, int max_sweeps, float tolerance, cudaStream_t stream);

}  // namespace soapb200
