// Building blocks of the blocked Householder QR that replaces the reference's SLATE geqrf/unmqr path
// (src/soap_tp/csrc/slate_bindings.cpp:125-189).
//
// The factorisation is organised so that all O(n^3) work is tensor-core GEMMs on operand planes
// (gemm_tf32x3.cu) and only the b-column panel is handled here:
//
//   qr_panel_kernel   cooperative kernel; every CTA keeps 256 rows of the panel in shared memory for
//                     the whole panel, so a column costs one fused pass (dot products of the pivot
//                     column with all other columns) + ONE grid-wide sync + one update pass.  The
//                     same dot products give, for columns left of the pivot, the entries v_j^T v_c
//                     that the compact-WY triangular factor needs -- no extra pass over V.
//   larft_kernel      T of H_0...H_{b-1} = I - V T V^T from those dot products (one CTA).
//   sum_partials / identity: small helpers for split-K partial sums and for Q's start value.
//
// Grid syncs are cooperative-groups syncs of a cooperative launch (no hand-written spin).
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "qr.h"

namespace cg = cooperative_groups;

namespace soapb200 {
namespace {

constexpr int kB = kQrPanelWidth;
constexpr int kRows = kQrRowsPerCta;
constexpr int kPanelThreads = 512;
constexpr int kPitch = kB + 1;

inline void check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

struct PanelArgs {
  const float* p_hi;
  const float* p_lo;
  int64_t ldp;
  int r, b;
  float* v_hi;
  float* v_lo;
  int64_t ldv;
  float* vt_hi;
  float* vt_lo;
  int64_t ldvt;
  float* tau;
  float* S;
  float* exchange;
};

__global__ void __launch_bounds__(kPanelThreads, 1) qr_panel_kernel(PanelArgs a) {
  extern __shared__ float smem[];
  float* P = smem;                       // [kRows][kPitch], unscaled reflector columns below the diagonal
  float* red = P + kRows * kPitch;       // [4][kB]
  float* dots = red + 4 * kB;            // [kB]   reduced dot products for the current pivot
  float* pivot_row = dots + kB;          // [kB]   row c of the panel
  float* scales = pivot_row + kB;        // [kB]   1 / (alpha - beta) of finished columns

  cg::grid_group grid = cg::this_grid();
  const int t = threadIdx.x;
  const int j = t & (kB - 1);
  const int q = t >> 7;                  // 0..3 : which 64-row slice of the CTA's rows
  const int row0 = blockIdx.x * kRows;   // first global row of this CTA
  const int rows_here = min(kRows, a.r - row0);
  const int ctas = gridDim.x;

  for (int idx = t; idx < kRows * kB; idx += kPanelThreads) {
    const int i = idx & (kRows - 1), jj = idx >> 8;   // consecutive threads -> consecutive rows (coalesced)
    float v = 0.f;
    if (i < rows_here && jj < a.b) {
      const int64_t off = (row0 + i) + static_cast<int64_t>(jj) * a.ldp;
      v = a.p_hi[off] + a.p_lo[off];
    }
    P[i * kPitch + jj] = v;
  }
  if (t < kB) scales[t] = 1.f;
  __syncthreads();

  float* partial = a.exchange;                               // [2][ctas][kB]
  float* rowbuf = a.exchange + 2 * static_cast<int64_t>(ctas) * kB;  // [2][kB]
  const int reflectors = min(a.b, a.r);

  for (int c = 0; c < reflectors; ++c) {
    const int parity = c & 1;
    // ---- pass 1: dot products of column c with every column over rows >= c ----
    {
      float acc = 0.f;
      const int lo_row = max(q * 64, c - row0);
      const int hi_row = min(q * 64 + 64, rows_here);
      for (int i = lo_row; i < hi_row; ++i) acc = fmaf(P[i * kPitch + j], P[i * kPitch + c], acc);
      red[q * kB + j] = acc;
    }
    __syncthreads();
    if (t < kB) {
      partial[(static_cast<int64_t>(parity) * ctas + blockIdx.x) * kB + t] =
          (red[t] + red[kB + t]) + (red[2 * kB + t] + red[3 * kB + t]);
      const int local_c = c - row0;
      if (local_c >= 0 && local_c < rows_here) rowbuf[parity * kB + t] = P[local_c * kPitch + t];
    }
    grid.sync();
    // ---- pass 2: Householder scalars (every CTA redundantly), update of the own rows ----
    if (t < kB) {
      float total = 0.f;
      for (int g = 0; g < ctas; ++g) total += __ldcg(&partial[(static_cast<int64_t>(parity) * ctas + g) * kB + t]);
      const float s = (t < c) ? scales[t] : 1.f;     // finished columns are stored unscaled
      dots[t] = total * s;
      pivot_row[t] = __ldcg(&rowbuf[parity * kB + t]) * s;
    }
    __syncthreads();
    const float alpha = pivot_row[c];
    const float normsq = dots[c];
    const float tail = normsq - alpha * alpha;
    float tau = 0.f, scale = 0.f;
    if (tail > 0.f && normsq > 0.f) {
      const float beta = -copysignf(sqrtf(normsq), alpha);
      tau = (beta - alpha) / beta;
      scale = 1.f / (alpha - beta);
    }
    // w_j = v_c^T column_j  (v_c = [1; scale * x_tail])
    const float w = pivot_row[j] + scale * (dots[j] - alpha * pivot_row[j]);
    if (blockIdx.x == 0 && q == 0) {
      if (j < c) a.S[j + static_cast<int64_t>(c) * kB] = w;
      if (j == c) a.tau[c] = tau;
    }
    if (j > c && tau != 0.f) {
      const float tw = tau * w;
      const int lo_row = max(q * 64, c - row0);
      const int hi_row = min(q * 64 + 64, rows_here);
      for (int i = lo_row; i < hi_row; ++i) {
        const float v = (row0 + i == c) ? 1.f : P[i * kPitch + c] * scale;
        P[i * kPitch + j] = fmaf(-tw, v, P[i * kPitch + j]);
      }
    }
    __syncthreads();
    if (t == 0) scales[c] = scale;
    __syncthreads();
  }

  // ---- outputs: V (r x b) and V^T (b x r) as operand planes ----
  for (int idx = t; idx < kRows * kB; idx += kPanelThreads) {
    const int i = idx & (kRows - 1), jj = idx >> 8;
    if (i < rows_here && jj < a.b) {
      const int gi = row0 + i;
      float v = 0.f;
      if (jj < reflectors) v = (gi > jj) ? P[i * kPitch + jj] * scales[jj] : (gi == jj ? 1.f : 0.f);
      const float h = tf32_rn(v);
      const int64_t off = gi + static_cast<int64_t>(jj) * a.ldv;
      a.v_hi[off] = h;
      a.v_lo[off] = v - h;
    }
  }
  for (int idx = t; idx < kRows * kB; idx += kPanelThreads) {
    const int jj = idx & (kB - 1), i = idx >> 7;       // consecutive threads -> consecutive columns (coalesced in V^T)
    if (i < rows_here && jj < a.b) {
      const int gi = row0 + i;
      float v = 0.f;
      if (jj < reflectors) v = (gi > jj) ? P[i * kPitch + jj] * scales[jj] : (gi == jj ? 1.f : 0.f);
      const float h = tf32_rn(v);
      const int64_t off = jj + static_cast<int64_t>(gi) * a.ldvt;
      a.vt_hi[off] = h;
      a.vt_lo[off] = v - h;
    }
  }
}

__global__ void __launch_bounds__(kB) larft_kernel(const float* __restrict__ S, const float* __restrict__ tau, int b,
                                                   float* t_hi, float* t_lo, float* tt_hi, float* tt_lo, int64_t ldt) {
  extern __shared__ float t_smem[];
  float (*T)[kPitch] = reinterpret_cast<float (*)[kPitch]>(t_smem);
  const int i = threadIdx.x;
  for (int c = 0; c < kB; ++c) T[i][c] = 0.f;
  __syncthreads();
  for (int c = 0; c < b; ++c) {
    const float tc = tau[c];
    float value = 0.f;
    if (i < c) {
      float acc = 0.f;
      for (int k = i; k < c; ++k) acc = fmaf(T[i][k], S[k + static_cast<int64_t>(c) * kB], acc);
      value = -tc * acc;
    } else if (i == c) {
      value = tc;
    }
    __syncthreads();
    T[i][c] = value;
    __syncthreads();
  }
  for (int c = 0; c < b; ++c) {
    if (i < b) {
      const float v = T[i][c];
      const float h = tf32_rn(v);
      t_hi[i + c * ldt] = h;          // T   column-major
      t_lo[i + c * ldt] = v - h;
      const float vt = T[c][i];       // T^T column-major
      const float ht = tf32_rn(vt);
      tt_hi[i + c * ldt] = ht;
      tt_lo[i + c * ldt] = vt - ht;
    }
  }
}

__global__ void sum_partials_kernel(const float* __restrict__ partials, int splits, int64_t stride, int64_t ld, float* hi,
                                    float* lo, int64_t ldp, int rows, int cols) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % rows);
    const int64_t c = idx / rows;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partials[s * stride + i + c * ld];
    const float h = tf32_rn(acc);
    hi[i + c * ldp] = h;
    lo[i + c * ldp] = acc - h;
  }
}

__global__ void identity_planes_kernel(float* hi, float* lo, int64_t ldp, int rows, int cols) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % rows);
    const int64_t c = idx / rows;
    hi[i + c * ldp] = (i == c) ? 1.f : 0.f;
    lo[i + c * ldp] = 0.f;
  }
}

inline int grid_for(int64_t total) {
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = 148 * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

void qr_panel(const float* p_hi, const float* p_lo, int64_t ldp, int r, int b, float* v_hi, float* v_lo, int64_t ldv,
              float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* S, float* exchange, cudaStream_t stream) {
  if (r <= 0 || b <= 0) return;
  if (b > kB) throw std::invalid_argument("qr_panel: panel wider than 128 columns");
  if (r > kQrMaxRows) throw std::invalid_argument("qr_panel: more rows than one cooperative grid can hold");
  const size_t smem = (static_cast<size_t>(kRows) * kPitch + 4 * kB + 3 * kB) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(qr_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) throw std::runtime_error(std::string("qr_panel attribute: ") + cudaGetErrorString(err));
    configured = true;
  }
  PanelArgs args{p_hi, p_lo, ldp, r, b, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, S, exchange};
  void* params[] = {&args};
  const int ctas = (r + kRows - 1) / kRows;
  cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(qr_panel_kernel), dim3(ctas), dim3(kPanelThreads),
                                                params, smem, stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("qr_panel launch: ") + cudaGetErrorString(err));
}

void qr_larft(const float* S, const float* tau, int b, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo, int64_t ldt,
              cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kB) * kPitch * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(larft_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) throw std::runtime_error(std::string("larft attribute: ") + cudaGetErrorString(err));
    configured = true;
  }
  larft_kernel<<<1, kB, smem, stream>>>(S, tau, b, t_hi, t_lo, tt_hi, tt_lo, ldt);
  check_launch("larft_kernel");
}

void sum_partials_to_planes(const float* partials, int splits, int64_t stride, int64_t ld, float* hi, float* lo,
                            int64_t ldp, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  sum_partials_kernel<<<grid_for(static_cast<int64_t>(rows) * cols), 256, 0, stream>>>(partials, splits, stride, ld, hi, lo,
                                                                                   ldp, rows, cols);
  check_launch("sum_partials_kernel");
}

void identity_planes(float* hi, float* lo, int64_t ldp, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  identity_planes_kernel<<<grid_for(static_cast<int64_t>(rows) * cols), 256, 0, stream>>>(hi, lo, ldp, rows, cols);
  check_launch("identity_planes_kernel");
}

}  // namespace soapb200
