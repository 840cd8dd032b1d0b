// Small symmetric eigenproblems of the two-sided block-Jacobi eigensolver.
//
// The eigensolver (engine/jacobi.py) replaces the reference's ELPA call
// (src/soap_tp/csrc/elpa_bindings.cpp:61-196) and its torch.linalg.eigh fallback
// (src/soap_tp/ops/factorizations.py:421-470).  It drives P to diagonal form by sweeps over pairs of
// 64-wide index blocks: for every pair the 128 x 128 diagonal block of the current matrix is
// diagonalised here, and the resulting orthogonal matrices are applied to the whole matrix (and to
// the accumulated eigenvectors) by batched tensor-core GEMMs.  One thread block per pair; the block and
// the accumulated rotations live in shared memory; parallel-order cyclic Jacobi (64 disjoint rotations
// per step, 127 steps per sweep) with an absolute threshold, so that nearly diagonal blocks -- the common
// case after the first outer sweeps -- cost one cheap sweep.  Rotation angles are computed in double
// precision so that each rotation is orthogonal to rounding and the product does not drift.
#include <stdexcept>
#include <string>

#include "jacobi.h"
#include "launch_util.h"

namespace soapb200 {
namespace {

constexpr int kN = 128;
constexpr int kPitch = kN + 1;
constexpr int kThreads = 512;

__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__global__ void __launch_bounds__(kThreads, 1)
jacobi_small_kernel(const float* __restrict__ s_hi, const float* __restrict__ s_lo, int64_t lds, float* u_hi, float* u_lo,
                    int64_t ldu, float* offdiag, float scale, int max_sweeps, float tolerance) {
  extern __shared__ float smem[];
  float (*Gs)[kPitch] = reinterpret_cast<float (*)[kPitch]>(smem);
  float (*Us)[kPitch] = reinterpret_cast<float (*)[kPitch]>(smem + kN * kPitch);
  __shared__ float cs[kN / 2], sn[kN / 2];
  __shared__ int pp[kN / 2], qq[kN / 2];
  __shared__ int rotated;
  __shared__ float block_max;

  const int t = threadIdx.x;
  const int batch = blockIdx.x;
  // diagonal block of the current matrix: entry (i, j) lives at planes[(128 b + i) * lds + 128 b + j]
  const int64_t origin = static_cast<int64_t>(batch) * kN * lds + static_cast<int64_t>(batch) * kN;
  for (int idx = t; idx < kN * kN; idx += kThreads) {
    const int j = idx & (kN - 1), i = idx >> 7;      // consecutive threads, consecutive j (contiguous in the planes)
    const int64_t off = origin + static_cast<int64_t>(i) * lds + j;
    Gs[i][j] = s_hi[off] + s_lo[off];
    Us[i][j] = (i == j) ? 1.f : 0.f;
  }
  if (t == 0) block_max = 0.f;
  __syncthreads();
  // symmetrise (the two triangles come from differently ordered sums) and measure the off-diagonal part
  float local_max = 0.f;
  for (int idx = t; idx < kN * kN; idx += kThreads) {
    const int i = idx & (kN - 1), j = idx >> 7;
    if (i > j) {
      const float v = 0.5f * (Gs[i][j] + Gs[j][i]);
      local_max = fmaxf(local_max, fabsf(v));
      Gs[i][j] = v;
    }
  }
  __syncthreads();
  for (int idx = t; idx < kN * kN; idx += kThreads) {
    const int i = idx & (kN - 1), j = idx >> 7;
    if (i < j) Gs[i][j] = Gs[j][i];
  }
  atomicMax(reinterpret_cast<int*>(&block_max), __float_as_int(local_max));   // non-negative floats order like ints
  __syncthreads();
  if (t == 0) atomicMax(reinterpret_cast<int*>(offdiag), __float_as_int(block_max / scale));
  const float threshold = tolerance * scale;

  for (int sweep = 0; sweep < max_sweeps; ++sweep) {
    if (t == 0) rotated = 0;
    __syncthreads();
    for (int step = 0; step < kN - 1; ++step) {
      // round-robin tournament over 128 indices: index 127 stays, the others rotate
      if (t < kN / 2) {
        int p, q;
        if (t == 0) {
          p = step;
          q = kN - 1;
        } else {
          p = (step + t) % (kN - 1);
          q = (step - t + (kN - 1)) % (kN - 1);
        }
        if (p > q) {
          const int tmp = p;
          p = q;
          q = tmp;
        }
        const float gpp = Gs[p][p], gqq = Gs[q][q], gpq = Gs[p][q];
        float c = 1.f, s = 0.f;
        if (fabsf(gpq) > threshold) {
          const double tau = (static_cast<double>(gqq) - gpp) / (2.0 * gpq);
          const double tt = (tau >= 0.0 ? 1.0 : -1.0) / (fabs(tau) + sqrt(1.0 + tau * tau));
          const double cd = 1.0 / sqrt(1.0 + tt * tt);
          c = static_cast<float>(cd);
          s = static_cast<float>(tt * cd);
          rotated = 1;
        }
        cs[t] = c;
        sn[t] = s;
        pp[t] = p;
        qq[t] = q;
      }
      __syncthreads();
      // columns: G <- G J, U <- U J
      for (int idx = t; idx < kN * (kN / 2); idx += kThreads) {
        const int r = idx & (kN - 1), pair = idx >> 7;
        const float c = cs[pair], s = sn[pair];
        if (s != 0.f) {
          const int p = pp[pair], q = qq[pair];
          const float gp = Gs[r][p], gq = Gs[r][q];
          Gs[r][p] = c * gp - s * gq;
          Gs[r][q] = s * gp + c * gq;
          const float up = Us[r][p], uq = Us[r][q];
          Us[r][p] = c * up - s * uq;
          Us[r][q] = s * up + c * uq;
        }
      }
      __syncthreads();
      // rows: G <- J^T G
      for (int idx = t; idx < kN * (kN / 2); idx += kThreads) {
        const int col = idx & (kN - 1), pair = idx >> 7;
        const float c = cs[pair], s = sn[pair];
        if (s != 0.f) {
          const int p = pp[pair], q = qq[pair];
          const float gp = Gs[p][col], gq = Gs[q][col];
          Gs[p][col] = c * gp - s * gq;
          Gs[q][col] = s * gp + c * gq;
        }
      }
      __syncthreads();
    }
    if (!rotated) break;
    __syncthreads();
  }
  // U as operand planes: element (k, n') at [k + (128 b + n') * ldu]
  for (int idx = t; idx < kN * kN; idx += kThreads) {
    const int k = idx & (kN - 1), n = idx >> 7;
    const float v = Us[k][n];
    const float h = tf32_rn(v);
    const int64_t off = k + (static_cast<int64_t>(batch) * kN + n) * ldu;
    u_hi[off] = h;
    u_lo[off] = v - h;
  }
}

}  // namespace

void jacobi_small(const float* s_hi, const float* s_lo, int64_t lds, int batches, float* u_hi, float* u_lo, int64_t ldu,
                  float* offdiag, float scale, int max_sweeps, float tolerance, cudaStream_t stream) {
  if (batches <= 0) return;
  const size_t smem = (2 * static_cast<size_t>(kN) * kPitch + 4) * sizeof(float);
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(jacobi_small_kernel), smem, configured, "jacobi_small");
  jacobi_small_kernel<<<batches, kThreads, smem, stream>>>(s_hi, s_lo, lds, u_hi, u_lo, ldu, offdiag, scale, max_sweeps,
                                                         tolerance);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("jacobi_small launch: ") + cudaGetErrorString(err));
}

}  // namespace soapb200
