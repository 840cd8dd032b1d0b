// Host-side interface of the Householder-tridiagonalisation eigensolver kernels (tridiag.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace soapb200 {

constexpr int kTridiagPanel = 32;   // reflectors per sytrd_panel launch (also half the GEMM K of the trailing update)

struct SytrdPanelArgs {
  float* A;            // n x n symmetric matrix, column-major, BOTH triangles kept; columns >= j0 are current
  int64_t lda;
  int n;
  int j0;              // first column of the panel
  int nb;              // columns in this launch (<= 32), j0 + nb <= n - 1
  float* vw;           // [2][64] scratch: the row of [V | W] that the next columns need from every CTA (double buffered)
  float* x;            // [n] scratch
  float* y;            // [n] scratch
  float* partial;      // [SM count][72] scratch
  double* d;           // [n] diagonal of T (written for columns of this panel; d[n-1] when `last`)
  double* e;           // [n-1] off-diagonal of T
  float* tau;          // [n-1]
  float* za_hi;        // operand planes of the trailing update, rows j0+nb .. n-1, 64 floats per row:
  float* za_lo;        //   Za row = [V | W], Zb row = [W | V]  ->  Za Zb^T = V W^T + W V^T
  float* zb_hi;
  float* zb_lo;
  float* v_hi;         // V (rows j0 .. n-1, nb columns; row j0 is zero) as planes, element (i - j0, c) at [i - j0 + c * ldv]
  float* v_lo;
  int64_t ldv;
  float* vt_hi;        // V^T as planes, element (c, i - j0) at [c + (i - j0) * ldvt]
  float* vt_lo;
  int64_t ldvt;
  float* t_hi;         // compact-WY factor T (H_j0 ... H_{j0+nb-1} = I - V T V^T) and T^T as planes, pitch ldt
  float* t_lo;
  float* tt_hi;
  float* tt_lo;
  int64_t ldt;
  unsigned int* barrier;   // one word of scratch for the grid barrier (cleared by the launcher)
  int* status;             // device status word
  int last;                // this is the last panel: also write d[n-1]
};

// Reduce columns j0 .. j0+nb-1 of the symmetric matrix to tridiagonal form (cooperative launch, one CTA per SM).
void sytrd_panel(const SytrdPanelArgs& args, cudaStream_t stream);

// lambda[k] = k-th smallest eigenvalue of the tridiagonal matrix (d, e) inside [lo, hi], by bisection (fp64).
void tridiagonal_bisect(const double* d, const double* e, int n, double lo, double hi, double pivmin, double* lambda,
                        cudaStream_t stream);

// z[i * n + k] = i-th entry of the unit eigenvector for lambda[n-1-k] (columns in descending eigenvalue order).
// lplus, dplus, uminus: scratch of n * n doubles each.
void tridiagonal_vectors(const double* d, const double* e, int n, const double* lambda, double pivmin, double* lplus,
                         double* dplus, double* uminus, float* z, cudaStream_t stream);

}  // namespace soapb200
