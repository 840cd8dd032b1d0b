// Building blocks of the blocked Householder QR that replaces the reference's SLATE geqrf/unmqr path
// (src/soap_tp/csrc/slate_bindings.cpp:125-189).
//
// The factorisation is organised so that all O(n^3) work is tensor-core GEMMs on operand planes
// (gemm_tf32x3.cu) and only the b-column panel is handled here:
//
//   qr_panel_kernel   cooperative kernel; every CTA keeps 256 rows of the panel in registers for
//                     the whole panel, so a column costs one sweep of dot products (pivot column
//                     with all other columns), ONE all-to-all exchange and one update sweep.  The
//                     same dot products give, for columns left of the pivot, the entries v_j^T v_c
//                     that the compact-WY triangular factor needs -- no extra pass over V.
//                     CTA 0 turns them into T of H_0...H_{b-1} = I - V T V^T while it waits.
//   sum_partials / identity: small helpers for split-K partial sums and for Q's start value.
//
// The panel's CTAs exchange partial dot products through packed {value, sequence} words with a
// bounded poll (cooperative launch guarantees co-residency).
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "qr.h"
#include "qr_device.cuh"

namespace soapb200 {
namespace {

using namespace qrdev;

inline void check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}


// Diagnostics that the default build leaves out: clock64 stamps of one column step of CTA 0 and switches that
// skip parts of the step (compile with -DSOAP_QR_TRACE; `kernel_cases panel --trace` needs such a build).
#ifdef SOAP_QR_TRACE
#define QR_STAMP(when, index) \
  do { if (a.trace && blockIdx.x == 0 && t == 0 && (when)) a.trace[(index)] = clock64(); } while (0)
#define QR_SKIP(bit) ((a.debug_skip & (bit)) != 0)
#else
#define QR_STAMP(when, index) do { } while (0)
#define QR_SKIP(bit) false
#endif

constexpr int kMaxPollWords = 10;   // words one thread requests per polling round (40 CTAs' worth per round)

constexpr int kSlice = 64 + 4;   // floats between the four 64-row slices of the pivot column in shared memory
                                 // (the 16-byte skew keeps the four lanes of a column on different banks)

// Panel factorisation.  The four lanes 4j .. 4j+3 of a warp own column j of the CTA's 256-row slab:
// lane q keeps rows q*64 .. q*64+63 in REGISTERS for the whole panel, so per-column reductions are
// two warp shuffles and shared memory only carries the pivot column.  A column step is
//   sweep 1  dot products of the pivot column with every column            (registers + shuffles)
//   exchange partial sums of all CTAs, every poll of the step in flight together; meanwhile CTA 0
//            builds column c-1 of the compact-WY factor T
//   barrier, Householder scalars (every thread), sweep 2: rank-1 update, next pivot column published
//   barrier
// i.e. two CTA barriers and one all-to-all per column.
__global__ void __launch_bounds__(kPanelThreads, 1) qr_panel_kernel(PanelArgs a) {
  __shared__ __align__(16) float xcol[2][4 * kSlice];   // pivot column (double buffered); rows above the pivot are zero
  __shared__ float pivot_stats[2][2];                   // {alpha, |x|^2} of the pivot column (double buffered)
  __shared__ float taus[kB];
  __shared__ float scol[kB];                            // column c of S = V^T V (entries above the diagonal)
  __shared__ float pivot_row_local[kB];                 // single-CTA launches: row c without a trip through memory
  __shared__ int abort_flag;
  extern __shared__ float dyn[];
  float (*T)[kPitch] = reinterpret_cast<float (*)[kPitch]>(dyn);   // CTA 0: compact-WY factor; all: output staging

  const int t = threadIdx.x;
  const int j = t >> 2;                  // column owned by this lane quad
  const int q = t & 3;                   // 64-row slice within the CTA's slab
  const int row0 = blockIdx.x * kRows;
  const int rows_here = min(kRows, a.r - row0);
  const int ctas = gridDim.x;
  const int my_first = q * 64;

  float P[64];
#pragma unroll
  for (int k = 0; k < 64; ++k) {
    const int i = my_first + k;
    float v = 0.f;
    if (i < rows_here && j < a.b) {
      const int64_t off = (row0 + i) + static_cast<int64_t>(j) * a.ldp;
      v = a.p_hi[off] + a.p_lo[off];
    }
    P[k] = v;
  }
  if (t < kB) taus[t] = 0.f;
  if (t == 0) abort_flag = 0;
  if (blockIdx.x == 0)
    for (int idx = t; idx < kB * kPitch; idx += kPanelThreads) dyn[idx] = 0.f;
  if (j == 0) {
#pragma unroll
    for (int k = 0; k < 64; ++k) xcol[0][q * kSlice + k] = P[k];   // column 0, pivot row 0: nothing above it
  }
  __syncthreads();

  const int reflectors = min(a.b, a.r);
  const unsigned int seq_base = a.epoch * 256u;
  float my_scale = 1.f;                  // 1 / (alpha - beta) of this lane's column once it has been a pivot

  for (int c = 0; c < reflectors; ++c) {
    const int parity = c & 1;
    const unsigned int seq = seq_base + static_cast<unsigned int>(c) + 1u;
    unsigned long long* slots = a.exchange + static_cast<int64_t>(parity) * (ctas + 1) * kB;
    const int pivot_local = c - row0;                   // local index of the pivot row (may be outside this CTA)
    const bool pivot_mine = pivot_local >= my_first && pivot_local < my_first + 64;
    QR_STAMP(c == 64, 7);
    // ---- sweep 1: dot product of the pivot column with this lane's slice of column j ----
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    {
      const float4* x4 = reinterpret_cast<const float4*>(&xcol[parity][q * kSlice]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) {
        const float4 x = x4[k4];
        acc0 = fmaf(P[4 * k4 + 0], x.x, acc0);
        acc1 = fmaf(P[4 * k4 + 1], x.y, acc1);
        acc2 = fmaf(P[4 * k4 + 2], x.z, acc2);
        acc3 = fmaf(P[4 * k4 + 3], x.w, acc3);
      }
    }
    float partial = (acc0 + acc1) + (acc2 + acc3);
    QR_STAMP(c == 64, 8);
    partial += __shfl_xor_sync(0xffffffffu, partial, 1);
    partial += __shfl_xor_sync(0xffffffffu, partial, 2);     // all four lanes: this CTA's partial dot for column j
    float row_value = 0.f;                                    // entry (c, j) of the panel, on the lane that holds it
    QR_STAMP(c == 64, 1);
    if (pivot_mine && !QR_SKIP(2)) row_value = take_pivot_entry(P, pivot_local - my_first, false);
    if (ctas > 1) {
      if (q == 0) ll_publish(&slots[static_cast<int64_t>(blockIdx.x) * kB + j], partial, seq);
      if (pivot_mine) ll_publish(&slots[static_cast<int64_t>(ctas) * kB + j], row_value, seq);
    }
    // ---- CTA 0, while the published words travel: column c-1 of T (four threads per row) ----
    QR_STAMP(c == 64, 2);
    if (blockIdx.x == 0 && c > 0 && !QR_SKIP(1)) t_column(T, scol, taus, c - 1, t);
    QR_STAMP(c == 64, 3);
    // ---- exchange: lane q polls the words of CTAs q, q+4, q+8, ... (index `ctas` = the pivot row) ----
    float total = partial, prow = row_value;
    if (ctas > 1) {
      float part = 0.f;
      prow = 0.f;
      bool failed = false;
      for (int base = 0; base <= ctas && !failed; base += 4 * kMaxPollWords) {
        unsigned long long words[kMaxPollWords];
        bool pending = true;
        unsigned int polls = 0;
        while (pending && polls < (1u << 20)) {
          pending = false;
#pragma unroll
          for (int u = 0; u < kMaxPollWords; ++u) {
            const int g = base + q + 4 * u;
            if (g <= ctas)
              asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];"
                           : "=l"(words[u]) : "l"(&slots[static_cast<int64_t>(g) * kB + j]) : "memory");
          }
#pragma unroll
          for (int u = 0; u < kMaxPollWords; ++u)
            if (base + q + 4 * u <= ctas && static_cast<unsigned int>(words[u] >> 32) != seq) pending = true;
          ++polls;
        }
        failed = pending;
#pragma unroll
        for (int u = 0; u < kMaxPollWords; ++u) {
          const int g = base + q + 4 * u;
          if (g < ctas) part += __uint_as_float(static_cast<unsigned int>(words[u]));
          else if (g == ctas) prow = __uint_as_float(static_cast<unsigned int>(words[u]));
        }
      }
      if (failed) {
        abort_flag = 1;
        atomicCAS(a.status, 0, kStatusPanelExchangeTimeout);
      }
      // fixed-shape reduction over the four lanes: identical on every CTA
      const float p1 = __shfl_xor_sync(0xffffffffu, part, 1);
      const float pair = (q & 1) ? (p1 + part) : (part + p1);
      const float p2 = __shfl_xor_sync(0xffffffffu, pair, 2);
      total = (q & 2) ? (p2 + pair) : (pair + p2);
      prow += __shfl_xor_sync(0xffffffffu, prow, 1);
      prow += __shfl_xor_sync(0xffffffffu, prow, 2);          // exactly one lane contributed a non-zero word
    } else {
      if (pivot_mine) pivot_row_local[j] = row_value;
    }
    if (ctas > 1 && j == c && q == 0) {
      pivot_stats[parity][0] = prow;
      pivot_stats[parity][1] = total;
    }
    if (ctas == 1 && j == c && q == 0) pivot_stats[parity][1] = total;
    QR_STAMP(c == 64, 6);
    __syncthreads();                                                              // barrier 1
    QR_STAMP(c == 64, 0);
    if (abort_flag) break;
    if (ctas == 1) prow = pivot_row_local[j];
    // finished columns are kept unscaled in the registers: apply their scale to the two dot-like values
    const float dots_j = total * ((j < c) ? my_scale : 1.f);
    const float prow_j = prow * ((j < c) ? my_scale : 1.f);
    const float alpha = (ctas == 1) ? pivot_row_local[c] : pivot_stats[parity][0];
    const float normsq = pivot_stats[parity][1];
    const float tail = normsq - alpha * alpha;
    float tau = 0.f, scale = 0.f;
    if (tail > 0.f && normsq > 0.f) {
      const float beta = -copysignf(sqrtf(normsq), alpha);
      tau = (beta - alpha) * __frcp_rn(beta);
      scale = __frcp_rn(alpha - beta);
    }
    const float w = prow_j + scale * (dots_j - alpha * prow_j);                   // v_c^T column_j
    if (j == c) my_scale = scale;
    if (blockIdx.x == 0 && q == 0) {
      if (j < c) scol[j] = w;
      if (j == c) {
        taus[c] = tau;
        a.tau[c] = tau;
      }
    }
    // ---- sweep 2: rank-1 update of the columns right of the pivot, publish the next pivot column ----
    if (j > c) {
      if (tau != 0.f) {
        const float tws = tau * w * scale;             // v_i = scale * x_i below the pivot
        const float4* x4 = reinterpret_cast<const float4*>(&xcol[parity][q * kSlice]);
#pragma unroll
        for (int k4 = 0; k4 < 16; ++k4) {
          const float4 x = x4[k4];
          P[4 * k4 + 0] = fmaf(-tws, x.x, P[4 * k4 + 0]);
          P[4 * k4 + 1] = fmaf(-tws, x.y, P[4 * k4 + 1]);
          P[4 * k4 + 2] = fmaf(-tws, x.z, P[4 * k4 + 2]);
          P[4 * k4 + 3] = fmaf(-tws, x.w, P[4 * k4 + 3]);
        }
      }
      // Row c right of the pivot now only holds R entries nobody reads again: zero them so that later
      // pivot columns leave the registers already masked above their pivot row.
      if (pivot_mine && !QR_SKIP(2)) take_pivot_entry(P, pivot_local - my_first, true);
      if (j == c + 1) {
        float4* x4 = reinterpret_cast<float4*>(&xcol[parity ^ 1][q * kSlice]);
#pragma unroll
        for (int k4 = 0; k4 < 16; ++k4) x4[k4] = make_float4(P[4 * k4], P[4 * k4 + 1], P[4 * k4 + 2], P[4 * k4 + 3]);
      }
    }
    __syncthreads();                                                              // barrier 2
    QR_STAMP(c == 64 || c == 63, c == 64 ? 4 : 5);
  }

  // ---- CTA 0: last column of T, then T and T^T as operand planes ----
  if (blockIdx.x == 0 && !abort_flag) {
    t_column(T, scol, taus, reflectors - 1, t);
    __syncthreads();
    for (int idx = t; idx < kB * kB; idx += kPanelThreads) {
      const int r = idx & (kB - 1), cidx = idx >> 7;
      if (r < a.b && cidx < a.b) {
        const float v = T[r][cidx];
        const float h = tf32_rn(v);
        a.t_hi[r + cidx * a.ldt] = h;
        a.t_lo[r + cidx * a.ldt] = v - h;
        const float vt = T[cidx][r];
        const float ht = tf32_rn(vt);
        a.tt_hi[r + cidx * a.ldt] = ht;
        a.tt_lo[r + cidx * a.ldt] = vt - ht;
      }
    }
    __syncthreads();
  }

  // ---- outputs: V (r x b) and V^T (b x r) through a shared-memory tile, one 64-row slice at a time ----
  const float out_scale = (j < reflectors) ? my_scale : 0.f;
#pragma unroll
  for (int k = 0; k < 64; ++k) {
    const int gi = row0 + my_first + k;
    float v = 0.f;
    if (j < reflectors) v = (gi > j) ? P[k] * out_scale : (gi == j ? 1.f : 0.f);
    P[k] = v;
  }
  float (*stage)[kPitch] = T;   // 64 x 129 staging tile (T has been written out)
  for (int slice = 0; slice < 4; ++slice) {
    __syncthreads();
    if (q == slice) {
#pragma unroll
      for (int k = 0; k < 64; ++k) stage[k][j] = P[k];
    }
    __syncthreads();
    for (int idx = t; idx < 64 * kB; idx += kPanelThreads) {
      const int k = idx & 63, jj = idx >> 6;             // consecutive threads -> consecutive rows (V)
      const int i = slice * 64 + k;
      if (i < rows_here && jj < a.b) {
        const float v = stage[k][jj];
        const float h = tf32_rn(v);
        const int64_t off = (row0 + i) + static_cast<int64_t>(jj) * a.ldv;
        a.v_hi[off] = h;
        a.v_lo[off] = v - h;
      }
    }
    for (int idx = t; idx < 64 * kB; idx += kPanelThreads) {
      const int jj = idx & (kB - 1), k = idx >> 7;       // consecutive threads -> consecutive columns (V^T)
      const int i = slice * 64 + k;
      if (i < rows_here && jj < a.b) {
        const float v = stage[k][jj];
        const float h = tf32_rn(v);
        const int64_t off = jj + static_cast<int64_t>(row0 + i) * a.ldvt;
        a.vt_hi[off] = h;
        a.vt_lo[off] = v - h;
      }
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

__global__ void identity_planes_kernel(float* hi, float* lo, int64_t ldp, int rows, int cols, int first_col) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % rows);
    const int64_t c = idx / rows;
    hi[i + c * ldp] = (i == c + first_col) ? 1.f : 0.f;
    lo[i + c * ldp] = 0.f;
  }
}

// out[c * ldo + k] = hi[k + c * ldp] + lo[k + c * ldp]: the fp32 matrix behind operand planes, each plane
// column written as one contiguous output row (planes of Q^T read out as Q).
__global__ void planes_sum_kernel(const float* __restrict__ hi, const float* __restrict__ lo, int64_t ldp, float* out,
                                  int64_t ldo, int depth, int cols) {
  const int64_t total = static_cast<int64_t>(depth) * cols;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(idx % depth);
    const int64_t c = idx / depth;
    out[c * ldo + k] = hi[k + c * ldp] + lo[k + c * ldp];
  }
}

inline int grid_for(int64_t total) {
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = 148 * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

unsigned int next_panel_epoch() {
  static unsigned int epoch = 0;
  epoch = (epoch + 1) & 0xFFFFFFu;
  if (epoch == 0) epoch = 1;
  return epoch;
}

void qr_panel(const float* p_hi, const float* p_lo, int64_t ldp, int r, int b, float* v_hi, float* v_lo, int64_t ldv,
              float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo,
              int64_t ldt, float* exchange, int* status, cudaStream_t stream, long long* trace, int debug_skip) {
  if (r <= 0 || b <= 0) return;
  if (b > kB) throw std::invalid_argument("qr_panel: panel wider than 128 columns");
  if (r > kQrMaxRows) throw std::invalid_argument("qr_panel: more rows than one cooperative grid can hold");
  const unsigned int epoch = next_panel_epoch();
  const size_t smem = static_cast<size_t>(kB) * kPitch * sizeof(float);
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(qr_panel_kernel), smem, configured, "qr_panel");
  PanelArgs args{p_hi, p_lo, ldp, r, b, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, t_hi, t_lo, tt_hi, tt_lo, ldt,
                 reinterpret_cast<unsigned long long*>(exchange), epoch, status, trace, debug_skip};
  void* params[] = {&args};
  const int ctas = (r + kRows - 1) / kRows;
  // Cooperative launch: the CTAs exchange data through global memory while running, so all of them
  // must be resident at the same time; the runtime refuses the launch otherwise.
  cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(qr_panel_kernel), dim3(ctas), dim3(kPanelThreads),
                                                params, smem, stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("qr_panel launch: ") + cudaGetErrorString(err));
}

void sum_partials_to_planes(const float* partials, int splits, int64_t stride, int64_t ld, float* hi, float* lo,
                            int64_t ldp, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  sum_partials_kernel<<<grid_for(static_cast<int64_t>(rows) * cols), 256, 0, stream>>>(partials, splits, stride, ld, hi, lo,
                                                                                   ldp, rows, cols);
  check_launch("sum_partials_kernel");
}

void identity_planes(float* hi, float* lo, int64_t ldp, int rows, int cols, cudaStream_t stream, int first_col) {
  if (rows <= 0 || cols <= 0) return;
  identity_planes_kernel<<<grid_for(static_cast<int64_t>(rows) * cols), 256, 0, stream>>>(hi, lo, ldp, rows, cols, first_col);
  check_launch("identity_planes_kernel");
}

void planes_sum(const float* hi, const float* lo, int64_t ldp, float* out, int64_t ldo, int depth, int cols,
                cudaStream_t stream) {
  if (depth <= 0 || cols <= 0) return;
  planes_sum_kernel<<<grid_for(static_cast<int64_t>(depth) * cols), 256, 0, stream>>>(hi, lo, ldp, out, ldo, depth, cols);
  check_launch("planes_sum_kernel");
}

}  // namespace soapb200
