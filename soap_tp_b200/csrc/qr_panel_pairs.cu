// Panel factorisation that retires TWO Householder columns per all-to-all exchange.
//
// The one-column kernel (qr.cu) is bound by its chain of exchanges: per column one sweep of dot
// products, one exchange between the CTAs, one update sweep.  Here a step takes the pivot columns
// x = a_c and y = a_{c+1} together:
//
//   sweep 1   D1_j = x . a_j and D2_j = y . a_j for every column j (one pass over the registers)
//   exchange  sums of D1, D2 over the CTAs and the pivot-row entries p1_j = a_j[c], p2_j = a_j[c+1]
//   scalars   H_c from (p1_c, D1_c) as before.  Everything H_{c+1} needs follows WITHOUT touching the
//             data again, because H_c is orthogonal:  with k = tau_c (v_c . y) and y' = H_c y,
//               y'[c]   = p1_{c+1} - k                      y'[c+1] = p2_{c+1} - k s_c p2_c
//               |y'|^2 over rows > c        = D2_{c+1} - y'[c]^2
//               y' . (H_c a_j) over rows >= c = D2_j
//             so v_{c+1} . (H_c a_j), the entries of V^T V that the compact-WY factor needs, and the
//             coefficients of the rank-2 update are per-column arithmetic on (D1_j, D2_j, p1_j, p2_j).
//   sweep 2   a_j <- a_j - A_j x - B_j y   (one pass), next two pivot columns published
//
// The subtraction D2_{c+1} - y'[c]^2 cancels when y is nearly parallel to x (rank-deficient input,
// repeated columns).  The step then retires column c only -- the decision is taken from exchanged
// sums that are bitwise identical on every CTA -- and column c + 1 becomes the next step's x, so
// the worst case is the one-column algorithm.  With the guard at half of |y|^2, rank-deficient,
// graded and duplicated inputs keep the orthogonality of Q at the one-column kernel's level (the NumPy
// restatement in utils/panel_pairs_reference.py shows 1e-3 without a guard, 2e-5 with a guard of 0.05).
//
// Register tiling, exchange words ({value, sequence} in 64 bits, bounded polls), T construction by
// CTA 0 in the shadow of the exchange and the output stage are those of qr.cu.
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "qr.h"
#include "qr_device.cuh"

namespace soapb200 {
namespace {

using namespace qrdev;

constexpr float kPairThreshold = 0.5f;    // |y'|^2 / |y|^2 below which the second column waits for the next step

// Extract (and optionally retire) entry `k` of a thread's register slice; `k` is warp-uniform, so the
// switch is one indirect branch instead of a chain of predicated selects.
#define SOAP_ENTRY_CASE(K) case K: if (K < kPer) { value = P[K < kPer ? K : 0]; if (clear) P[K < kPer ? K : 0] = 0.f; } break;
template <int kPer>
__device__ __forceinline__ float take_entry(float (&P)[kPer], int k, bool clear) {
  float value = 0.f;
  switch (k) {
    SOAP_ENTRY_CASE(0) SOAP_ENTRY_CASE(1) SOAP_ENTRY_CASE(2) SOAP_ENTRY_CASE(3) SOAP_ENTRY_CASE(4) SOAP_ENTRY_CASE(5)
    SOAP_ENTRY_CASE(6) SOAP_ENTRY_CASE(7) SOAP_ENTRY_CASE(8) SOAP_ENTRY_CASE(9) SOAP_ENTRY_CASE(10) SOAP_ENTRY_CASE(11)
    SOAP_ENTRY_CASE(12) SOAP_ENTRY_CASE(13) SOAP_ENTRY_CASE(14) SOAP_ENTRY_CASE(15) SOAP_ENTRY_CASE(16) SOAP_ENTRY_CASE(17)
    SOAP_ENTRY_CASE(18) SOAP_ENTRY_CASE(19) SOAP_ENTRY_CASE(20) SOAP_ENTRY_CASE(21) SOAP_ENTRY_CASE(22) SOAP_ENTRY_CASE(23)
    SOAP_ENTRY_CASE(24) SOAP_ENTRY_CASE(25) SOAP_ENTRY_CASE(26) SOAP_ENTRY_CASE(27) SOAP_ENTRY_CASE(28) SOAP_ENTRY_CASE(29)
    SOAP_ENTRY_CASE(30) SOAP_ENTRY_CASE(31) SOAP_ENTRY_CASE(32) SOAP_ENTRY_CASE(33) SOAP_ENTRY_CASE(34) SOAP_ENTRY_CASE(35)
    SOAP_ENTRY_CASE(36) SOAP_ENTRY_CASE(37) SOAP_ENTRY_CASE(38) SOAP_ENTRY_CASE(39) SOAP_ENTRY_CASE(40) SOAP_ENTRY_CASE(41)
    SOAP_ENTRY_CASE(42) SOAP_ENTRY_CASE(43) SOAP_ENTRY_CASE(44) SOAP_ENTRY_CASE(45) SOAP_ENTRY_CASE(46) SOAP_ENTRY_CASE(47)
    SOAP_ENTRY_CASE(48) SOAP_ENTRY_CASE(49) SOAP_ENTRY_CASE(50) SOAP_ENTRY_CASE(51) SOAP_ENTRY_CASE(52) SOAP_ENTRY_CASE(53)
    SOAP_ENTRY_CASE(54) SOAP_ENTRY_CASE(55) SOAP_ENTRY_CASE(56) SOAP_ENTRY_CASE(57) SOAP_ENTRY_CASE(58) SOAP_ENTRY_CASE(59)
    SOAP_ENTRY_CASE(60) SOAP_ENTRY_CASE(61) SOAP_ENTRY_CASE(62) SOAP_ENTRY_CASE(63)
    default: break;
  }
  return value;
}
#undef SOAP_ENTRY_CASE

__device__ __forceinline__ unsigned long long pack_word(float value, unsigned int seq) {
  return (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(value);
}

__device__ __forceinline__ void householder_scalars(float alpha, float normsq, float& tau, float& scale) {
  tau = 0.f;
  scale = 0.f;
  const float tail = normsq - alpha * alpha;
  if (tail > 0.f && normsq > 0.f) {
    const float beta = -copysignf(sqrtf(normsq), alpha);
    tau = (beta - alpha) * __frcp_rn(beta);
    scale = __frcp_rn(alpha - beta);
  }
}

// kPer rows of one column per thread: 64 (256-row CTAs, fewest SMs) or 32 (128-row CTAs: the sweeps are bound
// by shared-memory load latency, and with half the registers taken by the slab every load of a sweep can be in
// flight at once).
template <int kPer>
__global__ void __launch_bounds__(kPanelThreads, 1) qr_panel_pairs_kernel(PanelArgs a) {
  constexpr int kCtaRows = 4 * kPer;
  constexpr int kSlice = kPer + 4;     // floats between the four slices of a pivot column in shared memory
  constexpr int kVec = kPer / 4;       // 128-bit loads per sweep and pivot column
  constexpr int kPollPairs = kPer == 64 ? 7 : 17;   // 128-bit loads a thread keeps in flight per polling round
  __shared__ __align__(16) float xcol[2][4 * kSlice];   // pivot column c (double buffered); zero above the pivot row
  __shared__ __align__(16) float ycol[2][4 * kSlice];   // column c + 1 as it is before H_c is applied
  __shared__ float stats[2][8];                         // {p1_c, D1_c, p2_c, -, p1_c1, D1_c1, p2_c1, D2_c1}
  __shared__ float taus[kB];
  __shared__ float scol1[kB];                           // column c of S = V^T V (entries above the diagonal)
  __shared__ float scol2[kB];                           // column c + 1 of S
  __shared__ float row1_local[kB];                      // single-CTA launches: rows c and c + 1 without the exchange
  __shared__ float row2_local[kB];
  __shared__ int abort_flag;
  extern __shared__ float dyn[];
  float (*T)[kPitch] = reinterpret_cast<float (*)[kPitch]>(dyn);   // CTA 0: compact-WY factor; all: output staging

  const int t = threadIdx.x;
  const int j = t >> 2;                  // column owned by this lane quad
  const int q = t & 3;                   // 64-row slice within the CTA's slab
  const int row0 = blockIdx.x * kCtaRows;
  const int rows_here = min(kCtaRows, a.r - row0);
  const int ctas = gridDim.x;
  const int my_first = q * kPer;
  // The compact-WY factor T is built by the LAST CTA.  With more than one data CTA the host launches one
  // CTA more than the rows need: it owns no rows, publishes zeros at once and spends the time the others
  // sweep their slabs on T, so that no CTA the others wait for carries that work.
  const bool builds_t = blockIdx.x == gridDim.x - 1;
  const bool has_rows = rows_here > 0;

  float P[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
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
  if (builds_t)
    for (int idx = t; idx < kB * kPitch; idx += kPanelThreads) dyn[idx] = 0.f;
  if (j < 2) {
    float* dst = (j == 0) ? &xcol[0][q * kSlice] : &ycol[0][q * kSlice];
#pragma unroll
    for (int k = 0; k < kPer; ++k) dst[k] = P[k];
  }
  __syncthreads();

  const int reflectors = min(a.b, a.r);
  const unsigned int seq_base = a.epoch * 256u;
  float my_scale = 1.f;                  // 1 / (alpha - beta) of this lane's column once it has been a pivot
  int c = 0, step = 0;
  int built_c = -1, built_pair = 0;      // columns of T that CTA 0 still owes from the previous step

  while (c < reflectors) {
    const int parity = step & 1;
    const unsigned int seq = seq_base + static_cast<unsigned int>(step) + 1u;
    // [parity][ctas + 1][kB][2]: words {D1, D2} of every CTA, then {p1, p2} in row `ctas`
    unsigned long long* slots = a.exchange + static_cast<int64_t>(parity) * (ctas + 1) * kB * 2;
    const bool can_pair = c + 1 < reflectors;
    const bool row2_exists = c + 1 < a.r;
    const int local1 = c - row0 - my_first, local2 = c + 1 - row0 - my_first;
    const bool mine1 = local1 >= 0 && local1 < kPer;
    const bool mine2 = local2 >= 0 && local2 < kPer && row2_exists;

    // ---- sweep 1: dot products of both pivot columns with this lane's slice of column j ----
    float partial1 = 0.f, partial2 = 0.f;
    if (has_rows) {
      float x0 = 0.f, x1 = 0.f, x2 = 0.f, x3 = 0.f, y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
      const float4* x4 = reinterpret_cast<const float4*>(&xcol[parity][q * kSlice]);
      const float4* y4 = reinterpret_cast<const float4*>(&ycol[parity][q * kSlice]);
#pragma unroll
      for (int k4 = 0; k4 < kVec; ++k4) {
        const float4 x = x4[k4];
        const float4 y = y4[k4];
        x0 = fmaf(P[4 * k4 + 0], x.x, x0);
        x1 = fmaf(P[4 * k4 + 1], x.y, x1);
        x2 = fmaf(P[4 * k4 + 2], x.z, x2);
        x3 = fmaf(P[4 * k4 + 3], x.w, x3);
        y0 = fmaf(P[4 * k4 + 0], y.x, y0);
        y1 = fmaf(P[4 * k4 + 1], y.y, y1);
        y2 = fmaf(P[4 * k4 + 2], y.z, y2);
        y3 = fmaf(P[4 * k4 + 3], y.w, y3);
      }
      partial1 = (x0 + x1) + (x2 + x3);
      partial2 = (y0 + y1) + (y2 + y3);
    }
    partial1 += __shfl_xor_sync(0xffffffffu, partial1, 1);
    partial1 += __shfl_xor_sync(0xffffffffu, partial1, 2);
    partial2 += __shfl_xor_sync(0xffffffffu, partial2, 1);
    partial2 += __shfl_xor_sync(0xffffffffu, partial2, 2);   // all four lanes: this CTA's partial dots for column j
    float row1 = 0.f, row2 = 0.f;                             // entries (c, j) and (c + 1, j), on the lanes that hold them
    if (mine1) row1 = take_entry<kPer>(P, local1, false);
    if (mine2) row2 = take_entry<kPer>(P, local2, false);
    if (ctas > 1) {
      if (q == 0) {
        unsigned long long* mine = &slots[(static_cast<int64_t>(blockIdx.x) * kB + j) * 2];
        asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(mine), "l"(pack_word(partial1, seq)),
                     "l"(pack_word(partial2, seq))
                     : "memory");
      }
      unsigned long long* rows = &slots[(static_cast<int64_t>(ctas) * kB + j) * 2];
      if (mine1) ll_publish(rows, row1, seq);
      if (mine2) ll_publish(rows + 1, row2, seq);
    } else {
      if (mine1) row1_local[j] = row1;
      if (mine2) row2_local[j] = row2;
      if (!row2_exists && q == 0) row2_local[j] = 0.f;
    }

    // ---- CTA 0, while the published words travel: the columns of T the previous step produced ----
    if (builds_t && built_c >= 0) {
      t_column(T, scol1, taus, built_c, t);
      if (built_pair) {
        __syncthreads();
        t_column(T, scol2, taus, built_c + 1, t);
      }
    }

    // ---- exchange: lane q polls CTAs q, q+4, q+8, ... (index `ctas` holds the two pivot rows) ----
    float total1 = partial1, total2 = partial2, p1 = 0.f, p2 = 0.f;
    if (ctas > 1) {
      float part1 = 0.f, part2 = 0.f;
      bool failed = false;
      for (int base = 0; base <= ctas && !failed; base += 4 * kPollPairs) {
        unsigned long long w1[kPollPairs], w2[kPollPairs];
        bool pending = true;
        unsigned int polls = 0;
        while (pending && polls < (1u << 20)) {
          pending = false;
#pragma unroll
          for (int u = 0; u < kPollPairs; ++u) {
            const int g = base + q + 4 * u;
            if (g <= ctas)
              asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
                           : "=l"(w1[u]), "=l"(w2[u])
                           : "l"(&slots[(static_cast<int64_t>(g) * kB + j) * 2])
                           : "memory");
          }
#pragma unroll
          for (int u = 0; u < kPollPairs; ++u) {
            const int g = base + q + 4 * u;
            if (g <= ctas) {
              if (static_cast<unsigned int>(w1[u] >> 32) != seq) pending = true;
              if (static_cast<unsigned int>(w2[u] >> 32) != seq && (g < ctas || row2_exists)) pending = true;
            }
          }
          ++polls;
        }
        failed = pending;
#pragma unroll
        for (int u = 0; u < kPollPairs; ++u) {
          const int g = base + q + 4 * u;
          if (g < ctas) {
            part1 += __uint_as_float(static_cast<unsigned int>(w1[u]));
            part2 += __uint_as_float(static_cast<unsigned int>(w2[u]));
          } else if (g == ctas) {
            p1 = __uint_as_float(static_cast<unsigned int>(w1[u]));
            p2 = row2_exists ? __uint_as_float(static_cast<unsigned int>(w2[u])) : 0.f;
          }
        }
      }
      if (failed) {
        abort_flag = 1;
        atomicCAS(a.status, 0, kStatusPanelExchangeTimeout);
      }
      // fixed-shape reductions over the four lanes: identical on every CTA
      float o = __shfl_xor_sync(0xffffffffu, part1, 1);
      float pair_sum = (q & 1) ? (o + part1) : (part1 + o);
      o = __shfl_xor_sync(0xffffffffu, pair_sum, 2);
      total1 = (q & 2) ? (o + pair_sum) : (pair_sum + o);
      o = __shfl_xor_sync(0xffffffffu, part2, 1);
      pair_sum = (q & 1) ? (o + part2) : (part2 + o);
      o = __shfl_xor_sync(0xffffffffu, pair_sum, 2);
      total2 = (q & 2) ? (o + pair_sum) : (pair_sum + o);
      p1 += __shfl_xor_sync(0xffffffffu, p1, 1);
      p1 += __shfl_xor_sync(0xffffffffu, p1, 2);              // exactly one lane held the pivot-row words
      p2 += __shfl_xor_sync(0xffffffffu, p2, 1);
      p2 += __shfl_xor_sync(0xffffffffu, p2, 2);
    }
    if (q == 0 && j == c) {
      stats[parity][0] = p1;
      stats[parity][1] = total1;
      stats[parity][2] = p2;
    }
    if (q == 0 && j == c + 1) {
      stats[parity][4] = p1;
      stats[parity][5] = total1;
      stats[parity][6] = p2;
      stats[parity][7] = total2;
    }
    __syncthreads();                                                              // barrier 1
    if (abort_flag) break;
    if (ctas == 1) {
      p1 = row1_local[j];
      p2 = row2_local[j];
    }

    // ---- scalars of the step (every thread computes the same values) ----
    const float a1 = (ctas == 1) ? row1_local[c] : stats[parity][0];
    const float n1 = stats[parity][1];
    const float p2c = (ctas == 1) ? row2_local[c] : stats[parity][2];
    float t1, s1;
    householder_scalars(a1, n1, t1, s1);
    bool pair = false;
    float k = 0.f, yc = 0.f, yc1 = 0.f, t2 = 0.f, s2 = 0.f, p1c1 = 0.f, p2c1 = 0.f, d1c1 = 0.f;
    if (can_pair) {
      p1c1 = (ctas == 1) ? row1_local[c + 1] : stats[parity][4];
      d1c1 = stats[parity][5];
      p2c1 = (ctas == 1) ? row2_local[c + 1] : stats[parity][6];
      const float d2c1 = stats[parity][7];
      const float w1c1 = p1c1 + s1 * (d1c1 - a1 * p1c1);       // v_c . y
      k = t1 * w1c1;
      yc = p1c1 - k;
      yc1 = p2c1 - k * s1 * p2c;
      const float n2 = d2c1 - yc * yc;
      if (n2 > kPairThreshold * d2c1) {
        pair = true;
        householder_scalars(yc1, n2, t2, s2);
      }
    }
    // ---- this lane's column ----
    const float sj = (j < c) ? my_scale : 1.f;                  // finished columns are kept unscaled in the registers
    const float w1 = (p1 + s1 * (total1 - a1 * p1)) * sj;       // v_c . column_j
    float w2 = 0.f;
    if (pair) {
      if (j > c + 1) {                                          // v_{c+1} . (H_c a_j)
        const float ajc = p1 - t1 * w1;
        const float ajc1 = p2 - t1 * w1 * s1 * p2c;
        w2 = ajc1 + s2 * (total2 - yc * ajc - yc1 * ajc1);
      } else if (j < c) {                                       // v_{c+1} . v_j
        const float sum_y = total2 - p1c1 * p1 - p2c1 * p2;
        const float sum_x = total1 - a1 * p1 - p2c * p2;
        w2 = (p2 + s2 * (sum_y - k * s1 * sum_x)) * sj;
      } else if (j == c) {                                      // v_c . v_{c+1}
        const float sxy = (d1c1 - a1 * p1c1 - p2c * p2c1) - k * s1 * (n1 - a1 * a1 - p2c * p2c);
        w2 = s1 * p2c + s1 * s2 * sxy;
      }
    }
    if (j == c) my_scale = s1;
    if (pair && j == c + 1) my_scale = s2;
    if (builds_t && q == 0) {
      if (j < c) {
        scol1[j] = w1;
        scol2[j] = w2;
      }
      if (j == c) {
        scol2[c] = w2;
        taus[c] = t1;
        a.tau[c] = t1;
      }
      if (pair && j == c + 1) {
        taus[c + 1] = t2;
        a.tau[c + 1] = t2;
      }
    }

    // ---- sweep 2: a_j <- a_j - A x - B y for the columns right of c, next pivot columns published ----
    const int next = c + (pair ? 2 : 1);
    if (j > c && has_rows) {
      float B = 0.f;
      if (pair && j > c + 1) B = t2 * w2 * s2;
      const float A = t1 * w1 * s1 - B * k * s1;               // column c + 1 of a pair: y' = y - k s_c x (unscaled v)
      const float4* x4 = reinterpret_cast<const float4*>(&xcol[parity][q * kSlice]);
      if (pair) {
        const float4* y4 = reinterpret_cast<const float4*>(&ycol[parity][q * kSlice]);
#pragma unroll
        for (int k4 = 0; k4 < kVec; ++k4) {
          const float4 x = x4[k4];
          const float4 y = y4[k4];
          P[4 * k4 + 0] = fmaf(-B, y.x, fmaf(-A, x.x, P[4 * k4 + 0]));
          P[4 * k4 + 1] = fmaf(-B, y.y, fmaf(-A, x.y, P[4 * k4 + 1]));
          P[4 * k4 + 2] = fmaf(-B, y.z, fmaf(-A, x.z, P[4 * k4 + 2]));
          P[4 * k4 + 3] = fmaf(-B, y.w, fmaf(-A, x.w, P[4 * k4 + 3]));
        }
      } else if (A != 0.f) {
#pragma unroll
        for (int k4 = 0; k4 < kVec; ++k4) {
          const float4 x = x4[k4];
          P[4 * k4 + 0] = fmaf(-A, x.x, P[4 * k4 + 0]);
          P[4 * k4 + 1] = fmaf(-A, x.y, P[4 * k4 + 1]);
          P[4 * k4 + 2] = fmaf(-A, x.z, P[4 * k4 + 2]);
          P[4 * k4 + 3] = fmaf(-A, x.w, P[4 * k4 + 3]);
        }
      }
      // The pivot rows right of the pivots now hold R entries nobody reads again: zero them so that later
      // pivot columns leave the registers already masked above their pivot row.
      if (mine1) take_entry<kPer>(P, local1, true);
      if (pair && mine2) take_entry<kPer>(P, local2, true);
      if (j == next || j == next + 1) {
        float* dst = (j == next) ? &xcol[parity ^ 1][q * kSlice] : &ycol[parity ^ 1][q * kSlice];
        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int k4 = 0; k4 < kVec; ++k4) d4[k4] = make_float4(P[4 * k4], P[4 * k4 + 1], P[4 * k4 + 2], P[4 * k4 + 3]);
      }
    }
    __syncthreads();                                                              // barrier 2
    built_c = c;
    built_pair = pair ? 1 : 0;
    c = next;
    ++step;
  }

  if (a.trace && blockIdx.x == 0 && t == 0) a.trace[0] = step;   // diagnostics: exchange steps taken

  // ---- CTA 0: the columns of T of the last step, then T and T^T as operand planes ----
  if (builds_t && !abort_flag) {
    if (built_c >= 0) {
      t_column(T, scol1, taus, built_c, t);
      if (built_pair) {
        __syncthreads();
        t_column(T, scol2, taus, built_c + 1, t);
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

  // ---- outputs: V (r x b) and V^T (b x r) through a shared-memory tile, 64 rows at a time ----
  const float out_scale = (j < reflectors) ? my_scale : 0.f;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int gi = row0 + my_first + k;
    float v = 0.f;
    if (j < reflectors) v = (gi > j) ? P[k] * out_scale : (gi == j ? 1.f : 0.f);
    P[k] = v;
  }
  float (*stage)[kPitch] = T;   // 64 x 129 staging tile (T has been written out)
  constexpr int kLanesPerTile = 64 / kPer;    // quad lanes whose slices make up one 64-row tile
  for (int tile = 0; tile < kCtaRows / 64; ++tile) {
    __syncthreads();
    if (q / kLanesPerTile == tile) {
#pragma unroll
      for (int k = 0; k < kPer; ++k) stage[(q % kLanesPerTile) * kPer + k][j] = P[k];
    }
    __syncthreads();
    for (int idx = t; idx < 64 * kB; idx += kPanelThreads) {
      const int k = idx & 63, jj = idx >> 6;             // consecutive threads -> consecutive rows (V)
      const int i = tile * 64 + k;
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
      const int i = tile * 64 + k;
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

}  // namespace

namespace {

template <int kPer>
void launch_pairs(PanelArgs args, int r, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kB) * kPitch * sizeof(float);
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(qr_panel_pairs_kernel<kPer>), smem, configured, "qr_panel_pairs");
  void* params[] = {&args};
  int ctas = (r + 4 * kPer - 1) / (4 * kPer);
  if (ctas > 1 && ctas < 148) ++ctas;   // the rowless CTA that builds T (see the kernel)
  // Cooperative launch: the CTAs exchange data through global memory while running, so all of them
  // must be resident at the same time; the runtime refuses the launch otherwise.
  cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(qr_panel_pairs_kernel<kPer>), dim3(ctas),
                                                dim3(kPanelThreads), params, smem, stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("qr_panel_pairs launch: ") + cudaGetErrorString(err));
}

}  // namespace

void qr_panel_pairs(const float* p_hi, const float* p_lo, int64_t ldp, int r, int b, float* v_hi, float* v_lo, int64_t ldv,
                    float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi,
                    float* tt_lo, int64_t ldt, float* exchange, int* status, cudaStream_t stream, int rows_per_cta,
                    long long* steps_taken) {
  if (r <= 0 || b <= 0) return;
  if (b > kB) throw std::invalid_argument("qr_panel_pairs: panel wider than 128 columns");
  if (r > kQrMaxRows) throw std::invalid_argument("qr_panel_pairs: more rows than one cooperative grid can hold");
  if (rows_per_cta != 128 && rows_per_cta != 256) throw std::invalid_argument("qr_panel_pairs: rows_per_cta is 128 or 256");
  if (rows_per_cta == 128 && r > 148 * 128) rows_per_cta = 256;   // one CTA per SM at most
  const unsigned int epoch = next_panel_epoch();
  PanelArgs args{p_hi, p_lo, ldp, r, b, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, t_hi, t_lo, tt_hi, tt_lo, ldt,
                 reinterpret_cast<unsigned long long*>(exchange), epoch, status, steps_taken, 0};
  if (rows_per_cta == 128) launch_pairs<32>(args, r, stream);
  else launch_pairs<64>(args, r, stream);
}

}  // namespace soapb200
