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
  float* t_hi;                   // T and T^T of the compact WY form as operand planes (pitch ldt)
  float* t_lo;
  float* tt_hi;
  float* tt_lo;
  int64_t ldt;
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

// Extract (and retire) the pivot-row entry of this thread's register slab.  `k` is warp-uniform, so
// the switch is one indirect branch instead of 64 predicated selects.
#define SOAP_PIVOT_CASE(K) case K: value = P[K]; if (clear) P[K] = 0.f; break;
__device__ __forceinline__ float take_pivot_entry(float (&P)[64], int k, bool clear) {
  float value = 0.f;
  switch (k) {
    SOAP_PIVOT_CASE(0) SOAP_PIVOT_CASE(1) SOAP_PIVOT_CASE(2) SOAP_PIVOT_CASE(3) SOAP_PIVOT_CASE(4) SOAP_PIVOT_CASE(5)
    SOAP_PIVOT_CASE(6) SOAP_PIVOT_CASE(7) SOAP_PIVOT_CASE(8) SOAP_PIVOT_CASE(9) SOAP_PIVOT_CASE(10) SOAP_PIVOT_CASE(11)
    SOAP_PIVOT_CASE(12) SOAP_PIVOT_CASE(13) SOAP_PIVOT_CASE(14) SOAP_PIVOT_CASE(15) SOAP_PIVOT_CASE(16) SOAP_PIVOT_CASE(17)
    SOAP_PIVOT_CASE(18) SOAP_PIVOT_CASE(19) SOAP_PIVOT_CASE(20) SOAP_PIVOT_CASE(21) SOAP_PIVOT_CASE(22) SOAP_PIVOT_CASE(23)
    SOAP_PIVOT_CASE(24) SOAP_PIVOT_CASE(25) SOAP_PIVOT_CASE(26) SOAP_PIVOT_CASE(27) SOAP_PIVOT_CASE(28) SOAP_PIVOT_CASE(29)
    SOAP_PIVOT_CASE(30) SOAP_PIVOT_CASE(31) SOAP_PIVOT_CASE(32) SOAP_PIVOT_CASE(33) SOAP_PIVOT_CASE(34) SOAP_PIVOT_CASE(35)
    SOAP_PIVOT_CASE(36) SOAP_PIVOT_CASE(37) SOAP_PIVOT_CASE(38) SOAP_PIVOT_CASE(39) SOAP_PIVOT_CASE(40) SOAP_PIVOT_CASE(41)
    SOAP_PIVOT_CASE(42) SOAP_PIVOT_CASE(43) SOAP_PIVOT_CASE(44) SOAP_PIVOT_CASE(45) SOAP_PIVOT_CASE(46) SOAP_PIVOT_CASE(47)
    SOAP_PIVOT_CASE(48) SOAP_PIVOT_CASE(49) SOAP_PIVOT_CASE(50) SOAP_PIVOT_CASE(51) SOAP_PIVOT_CASE(52) SOAP_PIVOT_CASE(53)
    SOAP_PIVOT_CASE(54) SOAP_PIVOT_CASE(55) SOAP_PIVOT_CASE(56) SOAP_PIVOT_CASE(57) SOAP_PIVOT_CASE(58) SOAP_PIVOT_CASE(59)
    SOAP_PIVOT_CASE(60) SOAP_PIVOT_CASE(61) SOAP_PIVOT_CASE(62) SOAP_PIVOT_CASE(63)
    default: break;
  }
  return value;
}
#undef SOAP_PIVOT_CASE

constexpr int kMaxPollWords = 10;   // words one thread requests per polling round (40 CTAs' worth per round)

// Panel factorisation.  Thread (j, q) keeps rows q*64 .. q*64+63 of column j of its CTA's 256-row
// slab in REGISTERS for the whole panel; shared memory only carries the pivot column.  A column step
// is: dot products of the pivot column with every column (register sweep) -> one all-to-all exchange
// of the partial sums, all polls of a step in flight together -> Householder scalars -> rank-1
// update (register sweep).  While CTA 0 waits for the exchange its idle warps build the compact-WY
// triangular factor T column by column, so no separate pass over V is needed for it.
__global__ void __launch_bounds__(kPanelThreads, 1) qr_panel_kernel(PanelArgs a) {
  __shared__ __align__(16) float xcol[kRows];   // pivot column, zero at and above rows already eliminated
  __shared__ float red[4][kB];
  __shared__ float gathered[4][kB];             // per-quarter sums of the other CTAs' partial dot products
  __shared__ float dots[kB];
  __shared__ float pivot_row[kB];
  __shared__ float scales[kB];
  __shared__ float taus[kB];
  __shared__ float scol[kB];                    // column c of S = V^T V (entries above the diagonal)
  __shared__ int abort_flag;
  extern __shared__ float dyn[];
  float (*T)[kPitch] = reinterpret_cast<float (*)[kPitch]>(dyn);   // CTA 0: compact-WY factor; all: output staging

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
  if (t < kB) {
    scales[t] = 1.f;
    taus[t] = 0.f;
  }
  if (t == 0) abort_flag = 0;
  if (blockIdx.x == 0)
    for (int idx = t; idx < kB * kPitch; idx += kPanelThreads) dyn[idx] = 0.f;
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
    const bool pivot_mine = pivot_local >= my_first && pivot_local < my_first + 64;   // warp-uniform
    // ---- sweep 1: dot products of the pivot column with every column ----
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
    if (pivot_mine) {
      // Row c of the panel.  Right of the pivot it only holds R entries nobody reads again: they are
      // zeroed so that later pivot columns leave the registers already masked.
      const float row_value = take_pivot_entry(P, pivot_local - my_first, j > c);
      if (ctas > 1) ll_publish(&slots[static_cast<int64_t>(ctas) * kB + j], row_value, seq);
      else pivot_row[j] = row_value;
    }
    __syncthreads();                                                              // B1
    if (t < kB && ctas > 1)
      ll_publish(&slots[static_cast<int64_t>(blockIdx.x) * kB + t], (red[0][t] + red[1][t]) + (red[2][t] + red[3][t]), seq);
    // ---- CTA 0, warps 8..15, while the published words travel: column c-1 of T ----
    if (blockIdx.x == 0 && c > 0 && t >= 2 * kB) {
      const int cc = c - 1;
      const int i = (t - 2 * kB) >> 1, part = t & 1;      // two threads per row of T
      float acc = 0.f;
      if (i < cc)
        for (int k = i + part; k < cc; k += 2) acc = fmaf(T[i][k], scol[k], acc);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (part == 0) {
        if (i < cc) T[i][cc] = -taus[cc] * acc;
        else if (i == cc) T[i][cc] = taus[cc];
      }
    }
    // ---- exchange: quarter q of the threads polls the words of CTAs q, q+4, q+8, ... (and of the pivot
    //      row, index `ctas`); all words of a round are requested before any is inspected ----
    if (ctas > 1) {
      float part = 0.f;
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
          else if (g == ctas) pivot_row[j] = __uint_as_float(static_cast<unsigned int>(words[u]));
        }
      }
      if (failed) {
        abort_flag = 1;
        atomicCAS(a.status, 0, 4);
      }
      gathered[q][j] = part;
    }
    __syncthreads();                                                              // B2
    if (abort_flag) break;
    if (t < kB) {
      const float total = (ctas > 1) ? (gathered[0][t] + gathered[1][t]) + (gathered[2][t] + gathered[3][t])
                                     : (red[0][t] + red[1][t]) + (red[2][t] + red[3][t]);
      const float s = (t < c) ? scales[t] : 1.f;        // finished columns are kept unscaled
      dots[t] = total * s;
      pivot_row[t] *= s;
      if (t == 0 && pivot_local >= 0 && pivot_local < kRows) xcol[pivot_local] = 0.f;   // v_c[c] = 1 only touches dead R entries
    }
    __syncthreads();                                                              // B3
    const float alpha = pivot_row[c];
    const float normsq = dots[c];
    const float tail = normsq - alpha * alpha;
    float tau = 0.f, scale = 0.f;
    if (tail > 0.f && normsq > 0.f) {
      const float beta = -copysignf(sqrtf(normsq), alpha);
      tau = (beta - alpha) * __frcp_rn(beta);
      scale = __frcp_rn(alpha - beta);
    }
    const float w = pivot_row[j] + scale * (dots[j] - alpha * pivot_row[j]);   // v_c^T column_j
    if (blockIdx.x == 0 && q == 0) {
      if (j < c) scol[j] = w;
      if (j == c) {
        taus[c] = tau;
        a.tau[c] = tau;
        scales[c] = scale;
      }
    } else if (q == 0 && j == c) {
      scales[c] = scale;
    }
    // ---- sweep 2: rank-1 update of the columns right of the pivot, publish the next pivot column ----
    if (j > c && tau != 0.f) {
      const float tws = tau * w * scale;               // v_i = scale * x_i below the pivot, xcol is zero elsewhere
      const float4* x4 = reinterpret_cast<const float4*>(&xcol[my_first]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) {
        const float4 x = x4[k4];
        P[4 * k4 + 0] = fmaf(-tws, x.x, P[4 * k4 + 0]);
        P[4 * k4 + 1] = fmaf(-tws, x.y, P[4 * k4 + 1]);
        P[4 * k4 + 2] = fmaf(-tws, x.z, P[4 * k4 + 2]);
        P[4 * k4 + 3] = fmaf(-tws, x.w, P[4 * k4 + 3]);
      }
    }
    __syncthreads();                                                              // B4: everyone is done reading xcol
    if (j == c + 1) {   // rows above the new pivot were zeroed when their own pivot step finished
      float4* x4 = reinterpret_cast<float4*>(&xcol[my_first]);
#pragma unroll
      for (int k4 = 0; k4 < 16; ++k4) x4[k4] = make_float4(P[4 * k4], P[4 * k4 + 1], P[4 * k4 + 2], P[4 * k4 + 3]);
    }
    __syncthreads();                                                              // B5
  }

  // ---- CTA 0: last column of T, then T and T^T as operand planes ----
  if (blockIdx.x == 0 && !abort_flag) {
    const int cc = reflectors - 1;
    if (t >= 2 * kB) {
      const int i = (t - 2 * kB) >> 1, part = t & 1;
      float acc = 0.f;
      if (i < cc)
        for (int k = i + part; k < cc; k += 2) acc = fmaf(T[i][k], scol[k], acc);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (part == 0) {
        if (i < cc) T[i][cc] = -taus[cc] * acc;
        else if (i == cc) T[i][cc] = taus[cc];
      }
    }
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
  float (*stage)[kPitch] = T;   // 64 x 129 staging tile (T has been written out)
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
              float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo,
              int64_t ldt, float* exchange, int* status, cudaStream_t stream) {
  if (r <= 0 || b <= 0) return;
  if (b > kB) throw std::invalid_argument("qr_panel: panel wider than 128 columns");
  if (r > kQrMaxRows) throw std::invalid_argument("qr_panel: more rows than one cooperative grid can hold");
  static unsigned int epoch = 0;
  epoch = (epoch + 1) & 0xFFFFFFu;
  if (epoch == 0) epoch = 1;
  const size_t smem = static_cast<size_t>(kB) * kPitch * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t attr = cudaFuncSetAttribute(qr_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (attr != cudaSuccess) throw std::runtime_error(std::string("qr_panel attribute: ") + cudaGetErrorString(attr));
    configured = true;
  }
  PanelArgs args{p_hi, p_lo, ldp, r, b, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, t_hi, t_lo, tt_hi, tt_lo, ldt,
                 reinterpret_cast<unsigned long long*>(exchange), epoch, status};
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

void identity_planes(float* hi, float* lo, int64_t ldp, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  identity_planes_kernel<<<grid_for(static_cast<int64_t>(rows) * cols), 256, 0, stream>>>(hi, lo, ldp, rows, cols);
  check_launch("identity_planes_kernel");
}

}  // namespace soapb200
