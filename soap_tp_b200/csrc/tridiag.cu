// Symmetric eigensolver by Householder tridiagonalisation: the kernels.
//
// The reference's default basis initialisation is ELPA's one-stage solver, i.e. Householder reduction to
// tridiagonal form, a tridiagonal eigensolver and the back-transformation of the eigenvectors
// (src/soap_tp/csrc/elpa_bindings.cpp:61-196, called from src/soap_tp/ops/factorizations.py:472-547).  This file
// holds the three kernels of the same method here (driver: engine/tridiag.py):
//
//   sytrd_panel_kernel   32 columns of the reduction A -> Q^T A Q = T per launch (cooperative, one CTA per SM).
//                        Per column: the Householder vector v of the updated column, y = A v by streaming the
//                        trailing matrix once (every warp owns columns; A is kept with both triangles, so a
//                        column IS a row and all loads are contiguous), and w = tau (y - tau/2 (y.v) v) with
//                        the pending rank-2 updates of the panel applied implicitly.  Two grid barriers per
//                        column.  The deferred update A -= V W^T + W V^T is one tensor-core GEMM per panel
//                        (K = 64), for which the kernel leaves [V|W] and [W|V] as operand planes; it also
//                        leaves V, V^T and the compact-WY factor T in the formats of the QR panel kernel so
//                        that the back-transformation reuses the QR driver's products.
//   bisect_kernel        all eigenvalues of T by bisection on the Sturm count, one thread per eigenvalue, fp64.
//   twisted_kernel       one eigenvector per thread from the twisted factorisation of T - lambda I (forward
//                        and backward pivots, twist at the smallest |gamma|), fp64, written as fp32 columns.
//
// Every wait is bounded: the grid barrier gives up after 2^24 polls, poisons the counter so that all CTAs
// leave, and reports through the status word.
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "launch_util.h"
#include "status.h"
#include "tridiag.h"

namespace soapb200 {
namespace {

constexpr int kTB = kTridiagPanel;   // reflectors per launch
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kRowPitch = 2 * kTB;   // floats per row of the [V | W] store
constexpr unsigned int kPoison = 0x80000000u;

__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Barrier over all CTAs of a cooperative launch.  `target` is the counter value that means "everybody arrived".
__device__ __forceinline__ bool grid_barrier(unsigned int* counter, unsigned int& target, int* status) {
  __shared__ int gave_up;
  __syncthreads();
  target += gridDim.x;
  if (threadIdx.x == 0) {
    gave_up = 0;
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned int polls = 0;
    for (;;) {
      unsigned int seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
      if (seen & kPoison) { gave_up = 1; break; }
      if (static_cast<int>(seen - target) >= 0) break;
      if (++polls > (1u << 24)) {
        atomicOr(counter, kPoison);
        atomicCAS(status, 0, kStatusGridBarrierTimeout);
        gave_up = 1;
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  return gave_up == 0;
}

// Sum of one value per thread over the CTA, fixed order (warp shuffles, then the warps in index order).
__device__ __forceinline__ float block_sum(float v, float* scratch /* [kWarps] */) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) total += scratch[w];
  return total;
}

constexpr int kPartialPitch = kRowPitch + 8;   // floats per CTA in the partial-sum scratch

// Sum of slot `slot` of every CTA's partial sums, fixed order; all threads of the CTA call it and get the value.
__device__ __forceinline__ float sum_over_ctas(const float* partials, int slot, int ctas, float* broadcast) {
  if (threadIdx.x < 32) {
    float v = 0.f;
    for (int g = threadIdx.x; g < ctas; g += 32) v += __ldcg(&partials[static_cast<int64_t>(g) * kPartialPitch + slot]);
    v = warp_sum(v);
    if (threadIdx.x == 0) *broadcast = v;
  }
  __syncthreads();
  const float total = *broadcast;
  __syncthreads();
  return total;
}

// Row ownership: row i of the matrix (and of the panel's [V | W] store) belongs to CTA i % G, slot i / G.  A CTA keeps
// its rows of [V | W] in shared memory, so the row-wise phases never wait for L2; eight threads share a row.
constexpr int kRowSlots = kThreads / 8;          // rows handled per pass of a row-wise phase
constexpr int kStorePitch = kRowPitch + 1;       // floats per row of the shared store (odd: no bank conflicts)

__device__ __forceinline__ float octet_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__global__ void __launch_bounds__(kThreads, 1) sytrd_panel_kernel(SytrdPanelArgs a) {
  extern __shared__ __align__(16) float dyn[];   // v_s[n4] (the current Householder vector), then the row store
  __shared__ float red_w[kWarps][kRowPitch];     // partial sums of p = W^T v and q = V^T v
  __shared__ float pq[kRowPitch];                // q in [0, kTB), p in [kTB, 2 kTB)
  __shared__ float rowj[kRowPitch];              // row j of [V | W] while column j is being reduced
  __shared__ float scratch[kWarps];
  __shared__ float T[kTB][kTB + 1];              // CTA 0: compact-WY factor of the panel
  __shared__ float bcast;

  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int G = gridDim.x, b = blockIdx.x;
  const int n = a.n;
  const int64_t lda = a.lda;
  const int slots = (n + G - 1) / G;                          // rows of this CTA (some may be past the end)
  float* v_s = dyn;
  float* store = dyn + ((n + 3) & ~3);                        // [slots][kStorePitch]
  const int part = t & 7;                                     // which eighth of a row's coefficients
  const int gwarp = b * kWarps + warp, total_warps = G * kWarps;
  const bool vec_ok = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.A) & 15) == 0);
  unsigned int target = 0;
  float* partial = a.partial + static_cast<int64_t>(b) * kPartialPitch;

  if (b == 0)
    for (int idx = t; idx < kTB * (kTB + 1); idx += kThreads) (&T[0][0])[idx] = 0.f;
  for (int idx = t; idx < slots * kStorePitch; idx += kThreads) store[idx] = 0.f;
  if (t < kRowPitch) rowj[t] = 0.f;
  __syncthreads();

  // This thread's share of sum_c<k ( V[i][c] * second[kTB + c] + W[i][c] * second[c] ) for the row in `slot`; the
  // eight threads of the row add their shares with `octet_sum`, which every thread of the warp must reach.
  auto pending = [&](int slot, int k, const float* second) {
    const float* mine = store + slot * kStorePitch;
    float acc = 0.f;
    for (int c = part; c < k; c += 8) acc = fmaf(mine[c], second[kTB + c], fmaf(mine[kTB + c], second[c], acc));
    return acc;
  };

  // Column update of column `j` (k-th of the panel) for this CTA's rows (`rowj` holds row j of [V | W]): writes x,
  // the diagonal entry and this CTA's part of |x[j+2:]|^2.
  auto column_update = [&](int j, int k) {
    float sumsq = 0.f;
    for (int s0 = 0; s0 < slots; s0 += kRowSlots) {
      const int slot = s0 + (t >> 3);
      const int i = slot * G + b;
      const bool live = slot < slots && i >= j && i < n;
      const float correction = octet_sum(live ? pending(slot, k, rowj) : 0.f);
      if (live && part == 0) {
        const float value = a.A[i + static_cast<int64_t>(j) * lda] - correction;
        if (i == j) {
          a.d[j] = static_cast<double>(value);
        } else {
          a.x[i] = value;
          if (i > j + 1) sumsq = fmaf(value, value, sumsq);
        }
      }
    }
    const float cta_sumsq = block_sum(sumsq, scratch);
    if (t == 0) partial[0] = cta_sumsq;
  };

  column_update(a.j0, 0);
  bool alive = grid_barrier(a.barrier, target, a.status);

  for (int k = 0; k < a.nb && alive; ++k) {
    const int j = a.j0 + k;                      // column being reduced; its vector lives in rows j+1 .. n-1
    // ---- phase B: Householder scalars (every thread), v into shared memory, y = A v, partial p, q and y.v ----
    const float sigma = sum_over_ctas(a.partial, 0, G, &bcast);
    const float alpha = __ldcg(&a.x[j + 1]);
    float tau = 0.f, scale = 0.f, beta = alpha;
    if (sigma > 0.f) {
      beta = -copysignf(sqrtf(fmaf(alpha, alpha, sigma)), alpha);
      tau = (beta - alpha) / beta;
      scale = 1.f / (alpha - beta);
    }
    for (int i = t; i < n; i += kThreads) {
      float value = 0.f;
      if (i == j + 1) value = 1.f;
      else if (i > j + 1) value = __ldcg(&a.x[i]) * scale;
      v_s[i] = value;
    }
    __syncthreads();
    // q_c = sum_i V[i][c] v_i and p_c = sum_i W[i][c] v_i over this CTA's rows (thread = (coefficient, row group))
    {
      const int value = t % kRowPitch, group = t / kRowPitch;
      float acc = 0.f;
      if (value % kTB < k)
        for (int slot = group; slot < slots; slot += kThreads / kRowPitch) {
          const int i = slot * G + b;
          if (i > j && i < n) acc = fmaf(store[slot * kStorePitch + value], v_s[i], acc);
        }
      red_w[group][value] = acc;
    }
    __syncthreads();
    for (int slot = t; slot < slots; slot += kThreads) {         // V[:, k] = v for the own rows
      const int i = slot * G + b;
      if (i > j && i < n) store[slot * kStorePitch + k] = v_s[i];
    }
    // y = A[j+1:, j+1:] v: warp per column, lanes along the (contiguous) rows; y.v on the way
    float yv = 0.f;
    {
      const int first = j + 1;
      const int l0 = first & ~3;
      const int n4 = n & ~3;
      for (int c = first + gwarp; c < n; c += total_warps) {
        const float* col = a.A + static_cast<int64_t>(c) * lda;
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
        if (vec_ok) {
          int l = l0 + 4 * lane;
          for (; l + 384 < n4; l += 512) {
            const float4 m0 = __ldg(reinterpret_cast<const float4*>(col + l));
            const float4 m1 = __ldg(reinterpret_cast<const float4*>(col + l + 128));
            const float4 m2 = __ldg(reinterpret_cast<const float4*>(col + l + 256));
            const float4 m3 = __ldg(reinterpret_cast<const float4*>(col + l + 384));
            const float4 x0 = *reinterpret_cast<const float4*>(&v_s[l]);
            const float4 x1 = *reinterpret_cast<const float4*>(&v_s[l + 128]);
            const float4 x2 = *reinterpret_cast<const float4*>(&v_s[l + 256]);
            const float4 x3 = *reinterpret_cast<const float4*>(&v_s[l + 384]);
            acc0 = fmaf(m0.x, x0.x, acc0); acc0 = fmaf(m0.y, x0.y, acc0); acc0 = fmaf(m0.z, x0.z, acc0); acc0 = fmaf(m0.w, x0.w, acc0);
            acc1 = fmaf(m1.x, x1.x, acc1); acc1 = fmaf(m1.y, x1.y, acc1); acc1 = fmaf(m1.z, x1.z, acc1); acc1 = fmaf(m1.w, x1.w, acc1);
            acc2 = fmaf(m2.x, x2.x, acc2); acc2 = fmaf(m2.y, x2.y, acc2); acc2 = fmaf(m2.z, x2.z, acc2); acc2 = fmaf(m2.w, x2.w, acc2);
            acc3 = fmaf(m3.x, x3.x, acc3); acc3 = fmaf(m3.y, x3.y, acc3); acc3 = fmaf(m3.z, x3.z, acc3); acc3 = fmaf(m3.w, x3.w, acc3);
          }
          for (; l < n4; l += 128) {
            const float4 m0 = __ldg(reinterpret_cast<const float4*>(col + l));
            const float4 x0 = *reinterpret_cast<const float4*>(&v_s[l]);
            acc0 = fmaf(m0.x, x0.x, acc0); acc0 = fmaf(m0.y, x0.y, acc0); acc0 = fmaf(m0.z, x0.z, acc0); acc0 = fmaf(m0.w, x0.w, acc0);
          }
          for (int tail = n4 + lane; tail < n; tail += 32) acc1 = fmaf(__ldg(col + tail), v_s[tail], acc1);
        } else {
          for (int l = first + lane; l < n; l += 32) acc0 = fmaf(__ldg(col + l), v_s[l], acc0);
        }
        const float total = warp_sum((acc0 + acc1) + (acc2 + acc3));
        if (lane == 0) {
          a.y[c] = total;
          yv = fmaf(total, v_s[c], yv);
        }
      }
    }
    const float cta_yv = block_sum(yv, scratch);
    if (t < kRowPitch) {
      float total = 0.f;
      for (int g = 0; g < kThreads / kRowPitch; ++g) total += red_w[g][t];
      partial[1 + t] = total;
    }
    if (t == 0) partial[kRowPitch + 1] = cta_yv;
    if (!grid_barrier(a.barrier, target, a.status)) { alive = false; break; }

    // ---- phase C: p, q and s = y'.v over all CTAs; w for the own rows; then the update of the next column ----
    {
      const int value = t % kRowPitch, segment = t / kRowPitch;       // 512 threads = 64 values x 8 segments of CTAs
      float total = 0.f;
      for (int g = segment; g < G; g += kThreads / kRowPitch)
        total += __ldcg(&a.partial[static_cast<int64_t>(g) * kPartialPitch + 1 + value]);
      red_w[segment][value] = total;
      __syncthreads();
      if (t < kRowPitch) {
        float sum = 0.f;
        for (int seg = 0; seg < kThreads / kRowPitch; ++seg) sum += red_w[seg][t];
        pq[t] = sum;                               // q in [0, kTB), p in [kTB, 2 kTB)
      }
    }
    const float yv_raw = sum_over_ctas(a.partial, kRowPitch + 1, G, &bcast);    // (syncs: pq is visible after it)
    // y' = y - V p - W q, hence y'.v = y.v - q.p - p.q
    float qp = 0.f;
    for (int c = 0; c < k; ++c) qp = fmaf(pq[c], pq[kTB + c], qp);
    const float s = yv_raw - 2.f * qp;
    const float coef = -0.5f * tau * tau * s;
    for (int s0 = 0; s0 < slots; s0 += kRowSlots) {
      const int slot = s0 + (t >> 3);
      const int i = slot * G + b;
      const bool live = slot < slots && i > j && i < n;
      const float correction = octet_sum(live ? pending(slot, k, pq) : 0.f);      // V[i] . p + W[i] . q
      if (live && part == 0) {
        const float value = __ldcg(&a.y[i]) - correction;
        store[slot * kStorePitch + kTB + k] = fmaf(tau, value, coef * v_s[i]);    // w = tau y' - (tau^2 / 2) (y'.v) v
      }
    }
    if (b == 0) {
      // T[0:k, k] = -tau T[0:k, 0:k] q[0:k], T[k][k] = tau
      if (t < k) {
        float acc = 0.f;
        for (int c = t; c < k; ++c) acc = fmaf(T[t][c], pq[c], acc);
        T[t][k] = -tau * acc;
      }
      if (t == k) {
        T[k][k] = tau;
        a.tau[j] = tau;
        a.e[j] = static_cast<double>(beta);
      }
    }
    __syncthreads();
    // The row that the column after the next one needs from everybody is complete now up to this reflector: its
    // owner publishes it (two barriers lie between this store and its readers).
    {
      const int future = j + 2;
      if (k + 2 < a.nb && future < n && future % G == b && t < kRowPitch)
        a.vw[((k + 2) & 1) * kRowPitch + t] = store[(future / G) * kStorePitch + t];
    }
    if (k + 1 < a.nb) {
      // row j+1 of [V | W] for the next column: published entries for the older reflectors, rebuilt ones for this
      // one (v starts with 1 in row j+1; its w entry follows from y[j+1], p, q, which every CTA has)
      const int jn = j + 1;
      if (t < kRowPitch) {
        const int c = t % kTB;
        rowj[t] = (c < k) ? __ldcg(&a.vw[((k + 1) & 1) * kRowPitch + t]) : 0.f;
      }
      __syncthreads();
      if (t == 0) {
        float value = __ldcg(&a.y[jn]);
        for (int c = 0; c < k; ++c) value -= rowj[c] * pq[kTB + c] + rowj[kTB + c] * pq[c];
        rowj[k] = 1.f;
        rowj[kTB + k] = fmaf(tau, value, coef);
      }
      __syncthreads();
      column_update(jn, k + 1);
    }
    if (!grid_barrier(a.barrier, target, a.status)) { alive = false; break; }
  }
  if (!alive) return;

  const int next = a.j0 + a.nb;                    // first row / column of the trailing matrix
  // ---- outputs (every CTA for its own rows) ----
  if (a.last && (n - 1) % G == b && t == 0) {
    // d[n-1] = A[n-1][n-1] minus the panel's pending update of that entry
    const int i = n - 1;
    const float* mine = store + (i / G) * kStorePitch;
    float value = a.A[i + static_cast<int64_t>(i) * lda];
    for (int c = 0; c < a.nb; ++c) value -= 2.f * mine[c] * mine[kTB + c];
    a.d[i] = static_cast<double>(value);
  }
  for (int idx = t; idx < slots * kRowPitch; idx += kThreads) {
    const int slot = idx / kRowPitch, c = idx % kRowPitch;
    const int i = slot * G + b;
    if (i >= n) continue;
    const float* mine = store + slot * kStorePitch;
    if (i >= next) {
      // operand planes of the trailing update: Za row = [V | W], Zb row = [W | V]
      const int64_t base = static_cast<int64_t>(i - next) * kRowPitch;
      const float va = mine[c], vb = mine[(c + kTB) % kRowPitch];
      const float ha = tf32_rn(va), hb = tf32_rn(vb);
      a.za_hi[base + c] = ha;
      a.za_lo[base + c] = va - ha;
      a.zb_hi[base + c] = hb;
      a.zb_lo[base + c] = vb - hb;
    }
    if (i >= a.j0 && c < a.nb) {
      // V and V^T of the panel, rows j0 .. n-1 (row j0 is all zeros: every reflector starts below it; starting
      // there keeps the planes' first row on a 16-byte boundary)
      const int local = i - a.j0;
      const float v = mine[c];
      const float h = tf32_rn(v);
      a.v_hi[local + static_cast<int64_t>(c) * a.ldv] = h;
      a.v_lo[local + static_cast<int64_t>(c) * a.ldv] = v - h;
      a.vt_hi[c + static_cast<int64_t>(local) * a.ldvt] = h;
      a.vt_lo[c + static_cast<int64_t>(local) * a.ldvt] = v - h;
    }
  }
  if (b == 0) {
    for (int idx = t; idx < kTB * kTB; idx += kThreads) {
      const int r = idx % kTB, c = idx / kTB;
      const float v = (r < a.nb && c < a.nb) ? T[r][c] : 0.f;
      const float vt = (r < a.nb && c < a.nb) ? T[c][r] : 0.f;
      const float h = tf32_rn(v), ht = tf32_rn(vt);
      a.t_hi[r + c * a.ldt] = h;
      a.t_lo[r + c * a.ldt] = v - h;
      a.tt_hi[r + c * a.ldt] = ht;
      a.tt_lo[r + c * a.ldt] = vt - ht;
    }
  }
}

// ---- tridiagonal eigenvalues: bisection on the Sturm count ---------------------------------------------------
// d[0..n), e[0..n-1): diagonal and off-diagonal.  Thread k finds the k-th smallest eigenvalue inside [lo, hi].
__global__ void bisect_kernel(const double* __restrict__ d, const double* __restrict__ e, int n, double lo, double hi,
                              double pivmin, double* lambda) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  double left = lo, right = hi;
  for (int it = 0; it < 100; ++it) {
    const double mid = 0.5 * (left + right);
    if (mid <= left || mid >= right) break;
    int count = 0;                 // eigenvalues below mid = negative pivots of T - mid I = L D L^T
    double q = d[0] - mid;
    if (fabs(q) < pivmin) q = -pivmin;
    count += q < 0.0;
    for (int i = 1; i < n; ++i) {
      const double off = e[i - 1];
      q = d[i] - mid - off * off / q;
      if (fabs(q) < pivmin) q = -pivmin;
      count += q < 0.0;
    }
    if (count > k) right = mid; else left = mid;
  }
  lambda[k] = 0.5 * (left + right);
}

// ---- tridiagonal eigenvectors: twisted factorisation ---------------------------------------------------------
// Thread k handles eigenvalue lambda[n-1-k] (output column k, i.e. descending order).  Scratch: three arrays of
// n x n doubles laid out [i][k] so that the threads of a warp touch consecutive words.  Output: z[i * n + k], fp32.
__global__ void twisted_kernel(const double* __restrict__ d, const double* __restrict__ e, int n,
                               const double* __restrict__ lambda, double pivmin, double* lplus, double* dplus,
                               double* uminus, float* z) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const double lam = lambda[n - 1 - k];
  const int64_t ld = n;
  // forward: T - lam I = L+ D+ L+^T
  double dp = d[0] - lam;
  if (fabs(dp) < pivmin) dp = -pivmin;
  dplus[k] = dp;
  for (int i = 0; i + 1 < n; ++i) {
    const double l = e[i] / dp;
    lplus[i * ld + k] = l;
    dp = (d[i + 1] - lam) - l * e[i];
    if (fabs(dp) < pivmin) dp = -pivmin;
    dplus[(i + 1) * ld + k] = dp;
  }
  // backward: T - lam I = U- D- U-^T; gamma_i = D+_i + D-_i - (d_i - lam); twist where |gamma| is smallest
  double dm = d[n - 1] - lam;
  if (fabs(dm) < pivmin) dm = -pivmin;
  double best = fabs(dplus[(n - 1) * ld + k] + dm - (d[n - 1] - lam));
  int twist = n - 1;
  for (int i = n - 2; i >= 0; --i) {
    const double u = e[i] / dm;
    uminus[i * ld + k] = u;
    dm = (d[i] - lam) - u * e[i];
    if (fabs(dm) < pivmin) dm = -pivmin;
    const double gamma = fabs(dplus[i * ld + k] + dm - (d[i] - lam));
    if (gamma < best) { best = gamma; twist = i; }
  }
  // solve N z = e_twist: up with L+, down with U-; reuse dplus as the vector (it is no longer needed)
  double* vec = dplus;
  vec[twist * ld + k] = 1.0;
  double value = 1.0, sumsq = 1.0;
  for (int i = twist - 1; i >= 0; --i) {
    value = -lplus[i * ld + k] * value;
    vec[i * ld + k] = value;
    sumsq += value * value;
  }
  value = 1.0;
  for (int i = twist; i + 1 < n; ++i) {
    value = -uminus[i * ld + k] * value;
    vec[(i + 1) * ld + k] = value;
    sumsq += value * value;
  }
  const double inv = 1.0 / sqrt(sumsq);
  for (int i = 0; i < n; ++i) z[i * ld + k] = static_cast<float>(vec[i * ld + k] * inv);
}

}  // namespace

void sytrd_panel(const SytrdPanelArgs& args, cudaStream_t stream) {
  if (args.nb <= 0) return;
  if (args.nb > kTB) throw std::invalid_argument("sytrd_panel: at most 32 columns per launch");
  int device = 0, sms = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int ctas = sms > 0 ? sms : 1;     // one CTA per SM: all of them are resident, as the grid barrier needs
  // the Householder vector (n floats) and this CTA's rows of the panel's [V | W] store (ceil(n / CTAs) x 65 floats)
  const size_t smem = (static_cast<size_t>((args.n + 3) & ~3) + static_cast<size_t>((args.n + ctas - 1) / ctas) * (2 * kTB + 1)) *
                      sizeof(float);
  constexpr size_t kSmemLimit = 160 * 1024;
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(sytrd_panel_kernel), kSmemLimit, configured, "sytrd_panel");
  if (smem > kSmemLimit) throw std::invalid_argument("sytrd_panel: the matrix side is too large for one CTA's shared memory");
  cudaError_t err = cudaMemsetAsync(args.barrier, 0, sizeof(unsigned int), stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("sytrd_panel memset: ") + cudaGetErrorString(err));
  SytrdPanelArgs copy = args;
  void* params[] = {&copy};
  err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(sytrd_panel_kernel), dim3(ctas), dim3(kThreads), params, smem, stream);
  if (err != cudaSuccess) throw std::runtime_error(std::string("sytrd_panel launch: ") + cudaGetErrorString(err));
}

void tridiagonal_bisect(const double* d, const double* e, int n, double lo, double hi, double pivmin, double* lambda,
                        cudaStream_t stream) {
  if (n <= 0) return;
  bisect_kernel<<<(n + 63) / 64, 64, 0, stream>>>(d, e, n, lo, hi, pivmin, lambda);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("bisect_kernel: ") + cudaGetErrorString(err));
}

void tridiagonal_vectors(const double* d, const double* e, int n, const double* lambda, double pivmin, double* lplus,
                         double* dplus, double* uminus, float* z, cudaStream_t stream) {
  if (n <= 0) return;
  twisted_kernel<<<(n + 63) / 64, 64, 0, stream>>>(d, e, n, lambda, pivmin, lplus, dplus, uminus, z);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("twisted_kernel: ") + cudaGetErrorString(err));
}

}  // namespace soapb200
