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
//   larft_kernel      T of H_0...H_{b-1} = I - V T V^T from those dot products (one CTA).
//   sum_partials / identity: small helpers for split-K partial sums and for Q's start value.
//
// The panel's CTAs exchange partial dot products through packed {value, sequence} words with a
// bounded poll (cooperative launch guarantees co-residency).
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "qr.h"

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
  unsigned long long* exchange;  // [2][ctas + 1][kB] packed {value, sequence} words
  unsigned int epoch;            // distinguishes this launch's words from stale ones in `exchange`
  int* status;
};

// One 64-bit word carries a value and the sequence number that says which step it belongs to, so a
// reader learns "the data is there" and the data in the same load (one NVLink-free L2 round trip
// instead of flag-then-data).  Slots alternate by step parity; a CTA cannot run two steps ahead of
// another because it needs that CTA's word of the step in between.
__device__ __forceinline__ void ll_publish(unsigned long long* slot, float value, unsigned int seq) {
  const unsigned long long word = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(value);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(word) : "memory");
}
__device__ __forceinline__ bool ll_read(const unsigned long long* slot, unsigned int seq, float& value) {
  // Bounded: 2^22 polls of an L2-resident word is on the order of a second.
  for (unsigned int it = 0; it < (1u << 22); ++it) {
    unsigned long long word;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word) : "l"(slot) : "memory");
    if (static_cast<unsigned int>(word >> 32) == seq) {
      value = __uint_as_float(static_cast<unsigned int>(word));
      return true;
    }
  }
  return false;
}

// Panel factorisation.  Thread (j, q) keeps rows q*64 .. q*64+63 of column j of its CTA's 256-row
// slab in REGISTERS for the whole panel; shared memory only carries the pivot column, so a column
// step is two register sweeps (dot products, rank-1 update) around one all-to-all exchange.
__global__ void __launch_bounds__(kPanelThreads, 1) qr_panel_kernel(PanelArgs a) {
  __shared__ __align__(16) float xcol[kRows];   // pivot column, zero above the pivot row
  __shared__ __align__(16) float vcol[kRows];   // Householder vector of the current step
  __shared__ float red[4][kB];
  __shared__ float dots[kB];
  __shared__ float pivot_row[kB];
  __shared__ float scales[kB];
  __shared__ float stage[64][kB + 1];    // transpose staging for the V output
  __shared__ int abort_flag;

  const int t = threadIdx.x;
  const int j = t & (kB - 1);
  const int q = t >> 7;
  const int row0 = blockIdx.x * kRows;
  const int rows_here = min(kRows, a.r - row0);
  const int ctas = gridDim.x;
  const int my_first = q * 64;           // first local row held by this thread

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
  if (t < kB) scales[t] = 1.f;
  if (t == 0) abort_flag = 0;
  if (j == 0) {
#pragma unroll
    for (int k = 0; k < 64; ++k) xcol[my_first + k] = P[k];   // column 0, pivot row 0: nothing above it
  }
  __syncthreads();

  const int reflectors = min(a.b, a.r);
  const unsigned int seq_base = a.epoch * 256u;

  for (int c = 0; c < reflectors; ++c) {
    const int parity = c & 1;
    const unsigned int seq = seq_base + static_cast<unsigned int>(c) + 1u;
    unsigned long long* slots = a.exchange + static_cast<int64_t>(parity) * (ctas + 1) * kB;
    const int pivot_local = c - row0;                   // local index of the pivot row (may be outside this CTA)
    // ---- sweep 1: dot products of the pivot column with every column (rows above the pivot are zero in xcol) ----
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    {
      const float4* x4 = reinterpret_cast<const float4*>(&xcol[my_first]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) {
        const float4 x = x4[k4];
        acc0 = fmaf(P[4 * k4 + 0], x.x, acc0);
        acc1 = fmaf(P[4 * k4 + 1], x.y, acc1);
        acc2 = fmaf(P[4 * k4 + 2], x.z, acc2);
        acc3 = fmaf(P[4 * k4 + 3], x.w, acc3);
      }
    }
    red[q][j] = (acc0 + acc1) + (acc2 + acc3);
    if (pivot_local >= my_first && pivot_local < my_first + 64) {                  // row c of the panel (warp-uniform)
      float row_value = 0.f;
#pragma unroll
      for (int k = 0; k < 64; ++k) {
        if (my_first + k == pivot_local) {
          row_value = P[k];
          // right of the pivot, row c now only holds R entries nobody reads again: zero them so the
          // next pivot columns come out of the registers already masked
          if (j > c) P[k] = 0.f;
        }
      }
      if (ctas > 1) ll_publish(&slots[static_cast<int64_t>(ctas) * kB + j], row_value, seq);
      else pivot_row[j] = row_value;
    }
    __syncthreads();
    if (t < kB && ctas > 1)
      ll_publish(&slots[static_cast<int64_t>(blockIdx.x) * kB + t], (red[0][t] + red[1][t]) + (red[2][t] + red[3][t]), seq);
    // ---- exchange: every CTA sums all partial dot products in the same order ----
    if (t < kB) {
      float total = 0.f, prow = 0.f;
      bool ok = true;
      if (ctas == 1) {
        // one CTA: nothing to exchange, the reduced values are already in shared memory
        total = (red[0][t] + red[1][t]) + (red[2][t] + red[3][t]);
        prow = pivot_row[t];
      } else {
        // All words of a batch are requested before any is inspected, so the polls overlap instead
        // of paying one L2 round trip per CTA; the sum still runs in CTA order.
        constexpr int kBatch = 8;
        for (int base = 0; base < ctas + 1 && ok; base += kBatch) {
          unsigned long long words[kBatch];
          bool pending = true;
          unsigned int polls = 0;
          while (pending && polls < (1u << 20)) {
            pending = false;
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              if (base + u <= ctas)
                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];"
                             : "=l"(words[u]) : "l"(&slots[static_cast<int64_t>(base + u) * kB + t]) : "memory");
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              if (base + u <= ctas && static_cast<unsigned int>(words[u] >> 32) != seq) pending = true;
            ++polls;
          }
          ok = !pending;
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            if (base + u < ctas) total += __uint_as_float(static_cast<unsigned int>(words[u]));
            else if (base + u == ctas) prow = __uint_as_float(static_cast<unsigned int>(words[u]));
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(a.status, 0, 4);
      }
      const float s = (t < c) ? scales[t] : 1.f;        // finished columns are kept unscaled
      dots[t] = total * s;
      pivot_row[t] = prow * s;
    }
    __syncthreads();
    if (abort_flag) break;
    const float alpha = pivot_row[c];
    const float normsq = dots[c];
    const float tail = normsq - alpha * alpha;
    float tau = 0.f, scale = 0.f;
    if (tail > 0.f && normsq > 0.f) {
      const float beta = -copysignf(sqrtf(normsq), alpha);
      tau = (beta - alpha) / beta;
      scale = 1.f / (alpha - beta);
    }
    const float w = pivot_row[j] + scale * (dots[j] - alpha * pivot_row[j]);   // v_c^T column_j
    if (blockIdx.x == 0 && q == 0) {
      if (j < c) a.S[j + static_cast<int64_t>(c) * kB] = w;
      if (j == c) a.tau[c] = tau;
    }
    if (t < kRows) {
      const int gi = row0 + t;
      vcol[t] = (gi > c) ? xcol[t] * scale : 0.f;   // the unit entry at row c would only touch dead R entries
    }
    if (t == 0) scales[c] = scale;
    __syncthreads();
    // ---- sweep 2: rank-1 update of the columns right of the pivot, publish the next pivot column ----
    if (j > c && tau != 0.f) {
      const float tw = tau * w;
      const float4* v4 = reinterpret_cast<const float4*>(&vcol[my_first]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) {
        const float4 v = v4[k4];
        P[4 * k4 + 0] = fmaf(-tw, v.x, P[4 * k4 + 0]);
        P[4 * k4 + 1] = fmaf(-tw, v.y, P[4 * k4 + 1]);
        P[4 * k4 + 2] = fmaf(-tw, v.z, P[4 * k4 + 2]);
        P[4 * k4 + 3] = fmaf(-tw, v.w, P[4 * k4 + 3]);
      }
    }
    if (j == c + 1) {   // rows above the new pivot were zeroed when their own pivot step finished
      float4* x4 = reinterpret_cast<float4*>(&xcol[my_first]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) x4[k4] = make_float4(P[4 * k4], P[4 * k4 + 1], P[4 * k4 + 2], P[4 * k4 + 3]);
    }
    __syncthreads();
  }

  // ---- outputs: V^T (b x r) straight from registers, V (r x b) through a shared-memory transpose ----
  const float my_scale = (j < reflectors) ? scales[j] : 0.f;
#pragma unroll
  for (int k = 0; k < 64; ++k) {
    const int i = my_first + k;
    const int gi = row0 + i;
    float v = 0.f;
    if (j < reflectors) v = (gi > j) ? P[k] * my_scale : (gi == j ? 1.f : 0.f);
    P[k] = v;
    if (i < rows_here && j < a.b) {
      const float h = tf32_rn(v);
      const int64_t off = j + static_cast<int64_t>(gi) * a.ldvt;
      a.vt_hi[off] = h;
      a.vt_lo[off] = v - h;
    }
  }
  for (int slice = 0; slice < 4; ++slice) {
    __syncthreads();
    if (q == slice) {
#pragma unroll
      for (int k = 0; k < 64; ++k) stage[k][j] = P[k];
    }
    __syncthreads();
    for (int idx = t; idx < 64 * kB; idx += kPanelThreads) {
      const int k = idx & 63, jj = idx >> 6;             // consecutive threads -> consecutive rows
      const int i = slice * 64 + k;
      if (i < rows_here && jj < a.b) {
        const float v = stage[k][jj];
        const float h = tf32_rn(v);
        const int64_t off = (row0 + i) + static_cast<int64_t>(jj) * a.ldv;
        a.v_hi[off] = h;
        a.v_lo[off] = v - h;
      }
    }
  }
}

// T of the compact WY form, column by column: T[0:c, c] = -tau_c * T[0:c, 0:c] * S[0:c, c].
// 512 threads: four per row of T share each dot product.
__global__ void __launch_bounds__(512) larft_kernel(const float* __restrict__ S, const float* __restrict__ tau, int b,
                                                    float* t_hi, float* t_lo, float* tt_hi, float* tt_lo, int64_t ldt) {
  extern __shared__ float t_smem[];
  float (*T)[kPitch] = reinterpret_cast<float (*)[kPitch]>(t_smem);
  float (*Ss)[kPitch] = reinterpret_cast<float (*)[kPitch]>(t_smem + kB * kPitch);   // Ss[c][k] = S[k, c]
  __shared__ float taus[kB];
  const int t = threadIdx.x;
  for (int idx = t; idx < kB * kB; idx += 512) {
    const int k = idx & (kB - 1), c = idx >> 7;
    T[c][k] = 0.f;
    Ss[c][k] = (k < c && c < b) ? S[k + static_cast<int64_t>(c) * kB] : 0.f;
  }
  if (t < kB) taus[t] = (t < b) ? tau[t] : 0.f;
  __syncthreads();
  const int i = t >> 2, part = t & 3;
  for (int c = 0; c < b; ++c) {
    float acc = 0.f;
    if (i < c) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      int k = i + part;
      for (; k + 12 < c; k += 16) {
        a0 = fmaf(T[i][k], Ss[c][k], a0);
        a1 = fmaf(T[i][k + 4], Ss[c][k + 4], a1);
        a2 = fmaf(T[i][k + 8], Ss[c][k + 8], a2);
        a3 = fmaf(T[i][k + 12], Ss[c][k + 12], a3);
      }
      for (; k < c; k += 4) a0 = fmaf(T[i][k], Ss[c][k], a0);
      acc = (a0 + a1) + (a2 + a3);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    __syncthreads();
    if (part == 0) {
      if (i < c) T[i][c] = -taus[c] * acc;
      else if (i == c) T[i][c] = taus[c];
    }
    __syncthreads();
  }
  for (int idx = t; idx < kB * kB; idx += 512) {
    const int r = idx & (kB - 1), c = idx >> 7;
    if (r < b && c < b) {
      const float v = T[r][c];
      const float h = tf32_rn(v);
      t_hi[r + c * ldt] = h;          // T   column-major
      t_lo[r + c * ldt] = v - h;
      const float vt = T[c][r];       // T^T column-major
      const float ht = tf32_rn(vt);
      tt_hi[r + c * ldt] = ht;
      tt_lo[r + c * ldt] = vt - ht;
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
              float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* S, float* exchange, int* status,
              cudaStream_t stream) {
  if (r <= 0 || b <= 0) return;
  if (b > kB) throw std::invalid_argument("qr_panel: panel wider than 128 columns");
  if (r > kQrMaxRows) throw std::invalid_argument("qr_panel: more rows than one cooperative grid can hold");
  static unsigned int epoch = 0;
  epoch = (epoch + 1) & 0xFFFFFFu;
  if (epoch == 0) epoch = 1;
  PanelArgs args{p_hi, p_lo, ldp, r, b, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, S,
                 reinterpret_cast<unsigned long long*>(exchange), epoch, status};
  void* params[] = {&args};
  const int ctas = (r + kRows - 1) / kRows;
  // Cooperative launch: the CTAs exchange data through global memory while running, so all of them
  // must be resident at the same time; the runtime refuses the launch otherwise.
  cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(qr_panel_kernel), dim3(ctas), dim3(kPanelThreads),
                                                params, 0, stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("qr_panel launch: ") + cudaGetErrorString(err));
}

void qr_larft(const float* S, const float* tau, int b, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo, int64_t ldt,
              cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(2) * kB * kPitch * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(larft_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) throw std::runtime_error(std::string("larft attribute: ") + cudaGetErrorString(err));
    configured = true;
  }
  larft_kernel<<<1, 512, smem, stream>>>(S, tau, b, t_hi, t_lo, tt_hi, tt_lo, ldt);
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
