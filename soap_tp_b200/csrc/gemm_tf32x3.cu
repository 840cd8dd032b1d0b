// C = op(A^T B) on 5th-generation tensor cores with 3xTF32 error compensation.
//
// Problem form ("TN"): operands are column-major matrices Za (K x M) and Zb (K x N), i.e. both are
// K-contiguous, and the kernel forms acc[m, n] = sum_k Za[k, m] * Zb[k, n].  Every product of the
// SOAP pipeline is brought to this form by the caller (bases are kept in both orientations), so
// one kernel serves the rotations, the Gram updates and the power iteration.
//
// fp32-class accuracy on kind::tf32 hardware: each operand is supplied as two planes,
// hi = x with the 13 low mantissa bits cleared and lo = x - hi, prepared once per operand by
// split_planes_kernel (elementwise.cu).  Per 8-deep k-step the kernel issues three UMMAs,
// lo*hi + hi*lo + hi*hi, into one fp32 TMEM accumulator; the dropped lo*lo term is 2^-22 relative.
//
// Structure (one 128 x BN output tile per CTA, 192 threads):
//   warp 0, one lane : TMA producer  - four 128-byte-swizzled boxes per stage (A hi/lo, B hi/lo)
//   warp 1, one lane : MMA issuer    - tcgen05.mma.cta_group::1.kind::tf32, commit -> stage empty
//   warps 2..5       : epilogue      - tcgen05.ld 32x32b, fused store / EMA / Adam / split / mirror
// TMA zero-fills out-of-range rows and the K tail, so arbitrary M, N, K are handled by masking the
// stores only.  All waits are bounded (ptx.cuh).
//
// Replaces the SLATE gemm calls of the reference (src/soap_tp/csrc/slate_bindings.cpp:55-123 and
// :191-277), which run batched cuBLAS SGEMM on 128^3 tiles with MPI tile broadcasts in between.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>

#include "gemm.h"
#include "launch_util.h"
#include "ptx.cuh"

namespace soapb200 {

namespace {

constexpr int kBM = 128;
#ifndef SOAP_GEMM_BK
#define SOAP_GEMM_BK 32
#endif
// K extent of one pipeline stage: 32 fp32 = one 128-byte swizzle row (two 96 KB stages for 256-wide
// tiles) or 16 fp32 = one 64-byte swizzle row (four 48 KB stages).  Both were measured at 8192^3; the
// deeper pipeline of the 64-byte variant did not help (4.23 ms against 4.15 ms), because the kernel
// is bound by the L2 -> shared-memory traffic of the four operand planes, not by load latency.
constexpr int kBK = SOAP_GEMM_BK;
// Timing experiments only: SOAP_GEMM_TERMS < 3 drops correction products (wrong results, same data movement), which
// tells how much of the kernel's time is tensor-pipe time and how much is operand traffic.
#ifndef SOAP_GEMM_TERMS
#define SOAP_GEMM_TERMS 3
#endif
static_assert(kBK == 16 || kBK == 32, "one swizzle row per k-block: 64 or 128 bytes");
constexpr int kRowBytes = kBK * 4;
constexpr int kEpiWarps = 8;     // two warps per TMEM lane quarter, each owning half of the tile's columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
// The tensor core adds into its fp32 accumulator with truncation, so an accumulation that runs over
// the whole K extent drifts linearly in K (measured 6e-5 relative at K = 8192).  The accumulator is
// therefore drained every kPromote k-blocks: the epilogue warps add it, round-to-nearest, into a
// running sum held in registers while the tensor core fills the other TMEM buffer.
constexpr int kPromote = 64 / kBK;  // k-blocks (64 elements of K) accumulated inside TMEM before promotion

template <int BN>
struct TileConfig {
  static constexpr int kStageBytes = 2 * (kBM + BN) * kBK * 4;
  static constexpr int kStagesFit = (196 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesFit > 6 ? 6 : kStagesFit;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers (ping-pong)
  static constexpr int kColsPerThread = BN / 2;
};

struct alignas(64) GemmMaps {
  CUtensorMap a_hi, a_lo, b_hi, b_lo;     // MIXED: a_lo / b_lo describe the interleaved bf16 plane (hb | lb)
};

// Four consecutive rows of one column as bf16 (8 bytes).
__device__ __forceinline__ void store4_bf16(uint16_t* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = packed;
}
__device__ __forceinline__ uint16_t bf16_bits(float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&b);
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Global row / column of a local index.  symmetric == 1: the operands are whole matrices, indices are
// global already.  symmetric == 2: the output is this rank's packed block-cyclic part of a symmetric
// matrix; only entries on or below the GLOBAL diagonal are produced (the rest is pulled from the
// peers that own the mirrored entries).
__device__ __forceinline__ int global_row(const GemmProblem& p, int m) {
  if (p.symmetric != 2) return m;
  m += p.tri_m0;
  return ((m / p.tri_nb) * p.tri_Pr + p.tri_pr) * p.tri_nb + m % p.tri_nb;
}
__device__ __forceinline__ int global_col(const GemmProblem& p, int n) {
  if (p.symmetric != 2) return n;
  n += p.tri_n0;
  return ((n / p.tri_nb) * p.tri_Pc + p.tri_pc) * p.tri_nb + n % p.tri_nb;
}

// kEpiPush: where local element (m, n) goes in its consumers' planes.
struct PushTarget {
  int grid_row;      // pr' of the consuming ranks
  int64_t column;    // column of their gathered operand
};
__device__ __forceinline__ PushTarget push_target(const GemmProblem& p, int n) {
  const int jb = (n / p.push_nb) * p.push_Pc + p.push_pc;
  return PushTarget{jb % p.push_Pr, static_cast<int64_t>(jb / p.push_Pr) * p.push_nb + n % p.push_nb};
}
__device__ __forceinline__ int64_t push_depth(const GemmProblem& p, int m) {
  return static_cast<int64_t>((m / p.push_nb) * p.push_Pr + p.push_pr) * p.push_nb + m % p.push_nb;
}

constexpr int kTilePitch = kBM + 4;   // floats between columns of the staged tile (keeps 16-byte alignment)

struct Vec4 {
  float v[4];
};
__device__ __forceinline__ Vec4 load4(const float* p) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  return Vec4{{x.x, x.y, x.z, x.w}};
}
__device__ __forceinline__ void store4(float* p, const Vec4& x) {
  *reinterpret_cast<float4*>(p) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
}

// One output element (scalar path: ragged tiles, unaligned pitches, the diagonal band of symmetric products).
template <int MODE>
__device__ __forceinline__ void epilogue_scalar(const GemmProblem& prob, int64_t c_shift, int m, int n, float acc) {
  if constexpr (MODE == kEpiStore) {
    float* dst = prob.C + c_shift + m + static_cast<int64_t>(n) * prob.ldc;
    float v = prob.alpha * acc;
    if (prob.beta != 0.0f) v = fmaf(prob.beta, *dst, v);
    *dst = v;
    if (prob.symmetric == 1 && n < m) prob.C[c_shift + n + static_cast<int64_t>(m) * prob.ldc] = v;
  } else if constexpr (MODE == kEpiSplit) {
    const int64_t off = m + static_cast<int64_t>(n) * prob.ldp;
    float v = prob.alpha * acc;
    if (prob.beta != 0.0f) v = fmaf(prob.beta, prob.Chi[off] + prob.Clo[off], v);  // planes hold the old value
    const float hi = tf32_round(v);
    prob.Chi[off] = hi;
    if (prob.Chl) {
      const int64_t off16 = bf16_plane_index(m) + static_cast<int64_t>(n) * prob.ldp16;
      prob.Chl[off16] = bf16_bits(v);
      prob.Chl[off16 + 32] = bf16_bits(v - hi);
    } else {
      prob.Clo[off] = v - hi;
    }
    if (prob.C) prob.C[m + static_cast<int64_t>(n) * prob.ldc] = v;
  } else if constexpr (MODE == kEpiAdam) {
    float* mp = prob.mom + m + static_cast<int64_t>(n) * prob.ldm;
    float* vp = prob.var + m + static_cast<int64_t>(n) * prob.ldv;
    const float mo = fmaf(prob.beta1, *mp, (1.0f - prob.beta1) * acc);
    const float va = fmaf(prob.beta2, *vp, (1.0f - prob.beta2) * acc * acc);
    *mp = mo;
    *vp = va;
    const float u = (mo * prob.inv_bc1) / (sqrtf(va) * prob.inv_sqrt_bc2 + prob.eps);
    if (prob.Chi) {
      const int64_t off = m + static_cast<int64_t>(n) * prob.ldp;
      const float hi = tf32_round(u);
      prob.Chi[off] = hi;
      if (prob.Chl) {
        const int64_t off16 = bf16_plane_index(m) + static_cast<int64_t>(n) * prob.ldp16;
        prob.Chl[off16] = bf16_bits(u);
        prob.Chl[off16 + 32] = bf16_bits(u - hi);
      } else {
        prob.Clo[off] = u - hi;
      }
    }
    if (prob.C) prob.C[m + static_cast<int64_t>(n) * prob.ldc] = u;
  } else if constexpr (MODE == kEpiPush) {
    const PushTarget t = push_target(prob, n);
    const int64_t i = push_depth(prob, m);
    const float v = prob.alpha * acc;
    const float hi = tf32_round(v);
    for (int pc = 0; pc < prob.push_Pc; ++pc) {
      const uint64_t* entry = prob.push_table + 2 * (t.grid_row * prob.push_Pc + pc);
      reinterpret_cast<float*>(entry[0])[t.column * prob.push_ld + i] = hi;
      if (prob.push_mixed) {
        uint16_t* low = reinterpret_cast<uint16_t*>(entry[1]) + t.column * prob.push_ld16 + bf16_plane_index(i);
        low[0] = bf16_bits(v);
        low[32] = bf16_bits(v - hi);
      } else {
        reinterpret_cast<float*>(entry[1])[t.column * prob.push_ld + i] = v - hi;
      }
    }
  }
}

// Old values a column needs (the read half of the read-modify-write), four rows per lane.
template <int MODE>
__device__ __forceinline__ void epilogue_load4(const GemmProblem& prob, int64_t c_shift, int m, int n, Vec4& old0, Vec4& old1) {
  if constexpr (MODE == kEpiStore) {
    if (prob.beta != 0.0f) old0 = load4(prob.C + c_shift + m + static_cast<int64_t>(n) * prob.ldc);
  } else if constexpr (MODE == kEpiSplit) {
    if (prob.beta != 0.0f) {
      old0 = load4(prob.Chi + m + static_cast<int64_t>(n) * prob.ldp);
      old1 = load4(prob.Clo + m + static_cast<int64_t>(n) * prob.ldp);
    }
  } else if constexpr (MODE == kEpiAdam) {
    old0 = load4(prob.mom + m + static_cast<int64_t>(n) * prob.ldm);
    old1 = load4(prob.var + m + static_cast<int64_t>(n) * prob.ldv);
  }
}

template <int MODE>
__device__ __forceinline__ void epilogue_store4(const GemmProblem& prob, int64_t c_shift, int m, int n, const Vec4& acc,
                                                const Vec4& old0, const Vec4& old1) {
  if constexpr (MODE == kEpiStore) {
    Vec4 out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = prob.alpha * acc.v[i];
      if (prob.beta != 0.0f) v = fmaf(prob.beta, old0.v[i], v);
      out.v[i] = v;
    }
    store4(prob.C + c_shift + m + static_cast<int64_t>(n) * prob.ldc, out);
    if (prob.symmetric == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (n < m + i) prob.C[c_shift + n + static_cast<int64_t>(m + i) * prob.ldc] = out.v[i];
    }
  } else if constexpr (MODE == kEpiSplit) {
    Vec4 hi, lo, plain;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = prob.alpha * acc.v[i];
      if (prob.beta != 0.0f) v = fmaf(prob.beta, old0.v[i] + old1.v[i], v);
      plain.v[i] = v;
      hi.v[i] = tf32_round(v);
      lo.v[i] = v - hi.v[i];
    }
    store4(prob.Chi + m + static_cast<int64_t>(n) * prob.ldp, hi);
    if (prob.Chl) {
      uint16_t* dst = prob.Chl + bf16_plane_index(m) + static_cast<int64_t>(n) * prob.ldp16;
      store4_bf16(dst, plain.v);
      store4_bf16(dst + 32, lo.v);
    } else {
      store4(prob.Clo + m + static_cast<int64_t>(n) * prob.ldp, lo);
    }
    if (prob.C) store4(prob.C + m + static_cast<int64_t>(n) * prob.ldc, plain);
  } else if constexpr (MODE == kEpiAdam) {
    Vec4 mo, va, u, hi, lo;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float g = acc.v[i];
      mo.v[i] = fmaf(prob.beta1, old0.v[i], (1.0f - prob.beta1) * g);
      va.v[i] = fmaf(prob.beta2, old1.v[i], (1.0f - prob.beta2) * g * g);
      u.v[i] = (mo.v[i] * prob.inv_bc1) / (sqrtf(va.v[i]) * prob.inv_sqrt_bc2 + prob.eps);
      hi.v[i] = tf32_round(u.v[i]);
      lo.v[i] = u.v[i] - hi.v[i];
    }
    store4(prob.mom + m + static_cast<int64_t>(n) * prob.ldm, mo);
    store4(prob.var + m + static_cast<int64_t>(n) * prob.ldv, va);
    if (prob.Chi) {
      store4(prob.Chi + m + static_cast<int64_t>(n) * prob.ldp, hi);
      if (prob.Chl) {
        uint16_t* dst = prob.Chl + bf16_plane_index(m) + static_cast<int64_t>(n) * prob.ldp16;
        store4_bf16(dst, u.v);
        store4_bf16(dst + 32, lo.v);
      } else {
        store4(prob.Clo + m + static_cast<int64_t>(n) * prob.ldp, lo);
      }
    }
    if (prob.C) store4(prob.C + m + static_cast<int64_t>(n) * prob.ldc, u);
  } else if constexpr (MODE == kEpiPush) {
    // four consecutive local rows are four consecutive depth indices (block sizes are multiples of 4)
    const PushTarget t = push_target(prob, n);
    const int64_t i = push_depth(prob, m);
    Vec4 hi, lo, plain;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      plain.v[r] = prob.alpha * acc.v[r];
      hi.v[r] = tf32_round(plain.v[r]);
      lo.v[r] = plain.v[r] - hi.v[r];
    }
    for (int pc = 0; pc < prob.push_Pc; ++pc) {
      const uint64_t* entry = prob.push_table + 2 * (t.grid_row * prob.push_Pc + pc);
      store4(reinterpret_cast<float*>(entry[0]) + t.column * prob.push_ld + i, hi);
      if (prob.push_mixed) {
        uint16_t* low = reinterpret_cast<uint16_t*>(entry[1]) + t.column * prob.push_ld16 + bf16_plane_index(i);
        store4_bf16(low, plain.v);
        store4_bf16(low + 32, lo.v);
      } else {
        store4(reinterpret_cast<float*>(entry[1]) + t.column * prob.push_ld + i, lo);
      }
    }
  }
}

__device__ __forceinline__ bool aligned16(const void* p, int64_t pitch_floats) {
  return p == nullptr || (((reinterpret_cast<uintptr_t>(p) & 15) == 0) && (pitch_floats & 3) == 0);
}

// Fused epilogue over the staged tile (tile[n_local * kTilePitch + m_local]).  `ew` is the index of the
// calling warp among the kEpiWarps epilogue warps.
template <int BN, int MODE>
__device__ __forceinline__ void run_epilogue(const GemmProblem& prob, const float* tile, int m0, int n0, int ew, int lane,
                                             int64_t c_shift) {
  const int rows = min(kBM, prob.M - m0);
  const int cols = min(BN, prob.N - n0);
  if constexpr (MODE == kEpiRowMajor) {
    // one warp per output row, lanes sweep the columns so the stores are contiguous
    for (int r = ew; r < rows; r += kEpiWarps) {
      float* dst = prob.C + static_cast<int64_t>(m0 + r) * prob.ldc + n0;
      for (int n = lane; n < cols; n += 32) dst[n] = prob.alpha * tile[n * kTilePitch + r];
    }
    return;
  }
  bool vector = rows == kBM && !(prob.symmetric == 2 && ((prob.tri_nb | prob.tri_m0) & 3) != 0);
  if constexpr (MODE == kEpiStore) vector = vector && aligned16(prob.C + c_shift, prob.ldc);
  if (prob.Chl != nullptr) vector = vector && (prob.ldp16 & 3) == 0 && (reinterpret_cast<uintptr_t>(prob.Chl) & 7) == 0;
  if constexpr (MODE == kEpiSplit)
    vector = vector && aligned16(prob.Chi, prob.ldp) && aligned16(prob.Clo, prob.ldp) && aligned16(prob.C, prob.ldc);
  if constexpr (MODE == kEpiAdam)
    vector = vector && aligned16(prob.mom, prob.ldm) && aligned16(prob.var, prob.ldv) && aligned16(prob.Chi, prob.ldp) &&
             aligned16(prob.Clo, prob.ldp) && aligned16(prob.C, prob.ldc);
  if constexpr (MODE == kEpiPush)   // plane bases are segment starts (256-byte aligned); pitches and block size decide
    vector = vector && (prob.push_nb & 3) == 0 && (prob.push_ld & 3) == 0 && (prob.push_ld16 & 3) == 0;
  if (!vector) {
    for (int nl = ew; nl < cols; nl += kEpiWarps) {
      const int n = n0 + nl;
      for (int r = lane; r < rows; r += 32) {
        const int m = m0 + r;
        if (prob.symmetric && global_col(prob, n) > global_row(prob, m)) continue;
        epilogue_scalar<MODE>(prob, c_shift, m, n, tile[nl * kTilePitch + r]);
      }
    }
    return;
  }
  constexpr int kUnroll = 4;   // columns per warp whose loads are in flight together
  const int m = m0 + 4 * lane;
  const int gm = global_row(prob, m);   // the four rows of a lane are consecutive globally too (block sizes are multiples of 4)
  for (int base = ew * kUnroll; base < cols; base += kEpiWarps * kUnroll) {
    Vec4 old0[kUnroll], old1[kUnroll];
    int state[kUnroll];        // 0: skip, 1: vector, 2: element by element (diagonal band of a symmetric product)
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int nl = base + u, n = n0 + nl;
      state[u] = (nl < cols) ? 1 : 0;
      if (prob.symmetric && state[u]) {
        const int gn = global_col(prob, n);
        state[u] = (gn > gm + 3) ? 0 : (gn > gm ? 2 : 1);
      }
      old0[u] = old1[u] = Vec4{{0.f, 0.f, 0.f, 0.f}};
      if (state[u] == 1) epilogue_load4<MODE>(prob, c_shift, m, n, old0[u], old1[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int nl = base + u, n = n0 + nl;
      if (state[u] == 1) {
        epilogue_store4<MODE>(prob, c_shift, m, n, load4(tile + nl * kTilePitch + 4 * lane), old0[u], old1[u]);
      } else if (state[u] == 2) {
        const int gn = global_col(prob, n);
        for (int i = 0; i < 4; ++i)
          if (gn <= gm + i) epilogue_scalar<MODE>(prob, c_shift, m + i, n, tile[nl * kTilePitch + 4 * lane + i]);
      }
    }
  }
}

// Block-Jacobi pair update (N = 128): result column n' of batch item b becomes column
// c' = 64 * remap[2b + (n' >= 64)] + (n' & 63) of the next arrangement.  The result is written as
// operand planes in two orientations: (m, c') at [c' + m * ldp] (the operand of the next pair update)
// and, for rows m < m_limit, at [m + c' * ld2] (the operand of the next Gram product).
template <int BN>
__device__ __forceinline__ void run_pair_update(const GemmProblem& prob, const float* tile, int m0, int ew, int lane,
                                                int batch) {
  const int pos0 = prob.remap[2 * batch], pos1 = prob.remap[2 * batch + 1];
  const int rows = min(kBM, prob.M - m0);
  // orientation 1: one warp per result row, lanes along the result columns (runs of 32 contiguous floats)
  for (int r = ew; r < rows; r += kEpiWarps) {
    if (m0 + r < prob.o1_row_start) continue;
    const int64_t row_base = static_cast<int64_t>(m0 + r) * prob.ldp;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      const int nl = part * 32 + lane;
      const int dst = ((nl < 64) ? pos0 : pos1) * 64 + (nl & 63);
      const float v = tile[nl * kTilePitch + r];
      const float hi = tf32_round(v);
      prob.Chi[row_base + dst] = hi;
      prob.Clo[row_base + dst] = v - hi;
    }
  }
  // orientation 2: one warp per result column, four rows per lane
  if (prob.C2hi != nullptr && m0 < prob.m_limit && rows == kBM) {
    for (int nl = ew; nl < 128; nl += kEpiWarps) {
      const int dst = ((nl < 64) ? pos0 : pos1) * 64 + (nl & 63);
      const Vec4 v = load4(tile + nl * kTilePitch + 4 * lane);
      Vec4 hi, lo;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hi.v[i] = tf32_round(v.v[i]);
        lo.v[i] = v.v[i] - hi.v[i];
      }
      const int64_t off = (m0 + 4 * lane) + static_cast<int64_t>(dst) * prob.ld2;
      store4(prob.C2hi + off, hi);
      store4(prob.C2lo + off, lo);
    }
  }
}

template <int BN, int MODE, bool MIXED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmProblem prob, int* status) {
  // (the mixed variant needs the 32-element k-block build: 128-byte fp32 rows and 64-byte bf16 rows; the host refuses otherwise)
  using Cfg = TileConfig<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* acc_full = empty_bar + Cfg::kStages;   // [2] tensor core -> epilogue
  uint64_t* acc_empty = acc_full + 2;              // [2] epilogue -> tensor core
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Grouped raster: GROUP tile-rows share their B panels in L2 while they sweep the tile columns.
  const int tiles_m = (prob.M + kBM - 1) / kBM;
  const int tiles_n = (prob.N + BN - 1) / BN;
  constexpr int kGroup = 16;
  int tile_m, tile_n;
  {
    const int per_group = kGroup * tiles_n;
    const int group = blockIdx.x / per_group;
    const int first_m = group * kGroup;
    const int rows_in_group = min(kGroup, tiles_m - first_m);
    const int within = blockIdx.x % per_group;
    tile_m = first_m + within % rows_in_group;
    tile_n = within / rows_in_group;
  }
  const int m0 = tile_m * kBM;
  const int n0 = tile_n * BN;
  // Symmetric products: tiles strictly above the diagonal are produced by mirroring.
  if (prob.symmetric && global_col(prob, n0) > global_row(prob, min(m0 + kBM, prob.M) - 1)) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&maps.a_hi);
    tma_prefetch_descriptor(&maps.a_lo);
    tma_prefetch_descriptor(&maps.b_hi);
    tma_prefetch_descriptor(&maps.b_lo);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Split-K (kEpiStore only): blockIdx.y owns k-blocks [kb_first, kb_first + k_blocks) and writes its
  // own partial result at C + blockIdx.y * split_stride; the caller sums the partials in fixed order.
  const int total_k_blocks = (prob.K + kBK - 1) / kBK;
  const int per_split = (total_k_blocks + gridDim.y - 1) / gridDim.y;
  const int kb_first = blockIdx.y * per_split;
  const int k_blocks = max(0, min(total_k_blocks, kb_first + per_split) - kb_first);
  const int chunks = (k_blocks + kPromote - 1) / kPromote;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % Cfg::kStages;
      const uint32_t round = kb / Cfg::kStages;
      if (kb >= Cfg::kStages &&
          !mbar_wait_bounded(&empty_bar[s], (round - 1) & 1, abort_flag, status, kStatusSlotWaitTimeout))
        break;
      uint8_t* stage = smem + s * Cfg::kStageBytes;
      mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
      const int k0 = (kb_first + kb) * kBK;
      const int batch = blockIdx.z;
      const int ka = k0 + batch * prob.a_k_step, kbb = k0 + batch * prob.b_k_step;
      const int ra = m0 + batch * prob.a_row_step, rb = n0 + batch * prob.b_row_step;
      // MIXED: the second plane of each operand is the interleaved bf16 plane, 64 elements (128 bytes) per 32 of K
      const int ka2 = MIXED ? 2 * ka : ka, kbb2 = MIXED ? 2 * kbb : kbb;
      tma_load_2d(stage, &maps.a_hi, &full_bar[s], ka, ra);
      tma_load_2d(stage + kBM * kRowBytes, &maps.a_lo, &full_bar[s], ka2, ra);
      tma_load_2d(stage + 2 * kBM * kRowBytes, &maps.b_hi, &full_bar[s], kbb, rb);
      tma_load_2d(stage + 2 * kBM * kRowBytes + BN * kRowBytes, &maps.b_lo, &full_bar[s], kbb2, rb);
    }
    if (*abort_flag) {
      // give copies that are still in flight time to land before the CTA's shared memory is released
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = umma_idesc_tf32(kBM, BN);
    bool ok = true;
    int kb = 0;
    for (int c = 0; c < chunks && ok; ++c) {
      const int buf = c & 1;
      if (c >= 2) {
        ok = mbar_wait_bounded(&acc_empty[buf], ((c >> 1) - 1) & 1, abort_flag, status, kStatusAccumWaitTimeout);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(buf * BN);
      const int kb_end = min(k_blocks, kb + kPromote);
      for (int first = 1; kb < kb_end; ++kb) {
        const int s = kb % Cfg::kStages;
        const uint32_t round = kb / Cfg::kStages;
        ok = mbar_wait_bounded(&full_bar[s], round & 1, abort_flag, status, kStatusTmaWaitTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t stage = smem_u32(smem + s * Cfg::kStageBytes);
        if constexpr (MIXED) {
          constexpr uint32_t idesc16 = umma_idesc_bf16(kBM, BN);
          const uint64_t a_hi = umma_desc_kmajor<kRowBytes>(stage);
          const uint64_t a_hl = umma_desc_kmajor<kRowBytes>(stage + kBM * kRowBytes);
          const uint64_t b_hi = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes);
          const uint64_t b_hl = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes + BN * kRowBytes);
          // A 128-byte row of the bf16 plane: hb of the 32 k-elements in bytes 0..63, lb in bytes 64..127.  The two
          // correction products as bf16 MMAs (16 elements of K = 32 bytes each), then hi*hi in tf32.
          constexpr uint64_t kLb = 64 >> 4;
          // Even k-blocks issue the bf16 products first, odd ones the tf32 products, so that the tensor core changes
          // kind once per k-block instead of twice.
          const bool tf32_first = (kb & 1) != 0;
          if (tf32_first) {
#pragma unroll
            for (int k = 0; k < kBK / 8; ++k) {
              const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
              umma_tf32_ss(tmem_acc, a_hi + adv, b_hi + adv, idesc, first ? 0u : 1u);
              first = 0;
            }
          }
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
            umma_bf16_ss(tmem_acc, a_hl + kLb + adv, b_hl + adv, idesc16, first ? 0u : 1u);      // lo * hi
            first = 0;
            umma_bf16_ss(tmem_acc, a_hl + adv, b_hl + kLb + adv, idesc16, 1);                    // hi * lo
          }
          if (!tf32_first) {
#pragma unroll
            for (int k = 0; k < kBK / 8; ++k) {
              const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
              umma_tf32_ss(tmem_acc, a_hi + adv, b_hi + adv, idesc, 1);
            }
          }
          umma_commit(&empty_bar[s]);
          continue;
        }
        const uint64_t a_hi = umma_desc_kmajor<kRowBytes>(stage);
        const uint64_t a_lo = umma_desc_kmajor<kRowBytes>(stage + kBM * kRowBytes);
        const uint64_t b_hi = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes);
        const uint64_t b_lo = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes + BN * kRowBytes);
#pragma unroll
        for (int k = 0; k < kBK / 8; ++k) {
          const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);  // 8 tf32 = 32 bytes along the swizzle row
          // small terms first, the dominant hi*hi product last
#if SOAP_GEMM_TERMS >= 3
          umma_tf32_ss(tmem_acc, a_lo + adv, b_hi + adv, idesc, first ? 0u : 1u);
          first = 0;
#endif
#if SOAP_GEMM_TERMS >= 2
          umma_tf32_ss(tmem_acc, a_hi + adv, b_lo + adv, idesc, first ? 0u : 1u);
          first = 0;
#endif
          umma_tf32_ss(tmem_acc, a_hi + adv, b_hi + adv, idesc, first ? 0u : 1u);
          first = 0;
        }
        umma_commit(&empty_bar[s]);  // stage reusable once these UMMAs have read it
      }
      if (ok) umma_commit(&acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ---------------- promotion + epilogue ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;              // TMEM lane quarter this warp may read
    const int half = ew >> 2;                  // which half of the tile's columns
    constexpr int kCols = Cfg::kColsPerThread;
    const int col0 = half * kCols;
    float sum[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) sum[j] = 0.0f;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int buf = c & 1;
      ok = mbar_wait_bounded(&acc_full[buf], (c >> 1) & 1, abort_flag, status, kStatusAccumWaitTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * BN + col0);
#pragma unroll
      for (int cc = 0; cc < kCols; cc += 32) {
        uint32_t raw[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(cc), raw);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[cc + j] += __uint_as_float(raw[j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    // Stage the running sums in shared memory (the pipeline stages are idle once the last chunk has
    // been drained) and run the fused epilogue as a compact rolled loop: one warp per output column,
    // 16 bytes per lane.  Keeping the epilogue out of the 128-fold unrolled register code matters:
    // straight-line code that long is fetched once per tile and stalls on instruction fetch.
    float* tile = reinterpret_cast<float*>(smem);
    {
      const int m_local = quarter * 32 + lane;
#pragma unroll
      for (int jx = 0; jx < kCols; ++jx) tile[(col0 + jx) * kTilePitch + m_local] = sum[jx];
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kEpiWarps * 32) : "memory");
    if (ok) {
      const int64_t c_shift = ((gridDim.y > 1) ? static_cast<int64_t>(blockIdx.y) * prob.split_stride : 0) +
                              static_cast<int64_t>(blockIdx.z) * prob.c_batch_stride;
      if constexpr (MODE == kEpiPairUpdate) run_pair_update<BN>(prob, tile, m0, ew, lane, blockIdx.z);
      else run_epilogue<BN, MODE>(prob, tile, m0, n0, ew, lane, c_shift);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// The same product on CTA pairs (`cta_group::2`): the two CTAs of a cluster compute a 256 x 256 tile together.  Each CTA
// stages its own 128 rows of A and HALF of the 256 rows of B (each with its own TMA, no multicast), the leader CTA issues
// M = 256 MMAs that read both CTAs' shared memory, and each CTA's TMEM receives its own 128 x 256 half of the
// accumulator, which it promotes and stores exactly as the single-CTA kernel does.  Per k-block a CTA therefore loads
// 64 KB instead of 96 KB: operand traffic from L2 into shared memory, which is what bounds the single-CTA kernel once the
// correction products run as bf16 MMAs, drops by a third, and three stages fit instead of two.
constexpr int kPairStages = 3;
constexpr int kPairStageBytes = 2 * (kBM + 128) * kBK * 4;       // A (hi, second plane) + half of B (hi, second plane)
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr int kPairBN = 256;

template <int MODE, bool MIXED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmProblem prob, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);   // used in the leader CTA only
  uint64_t* empty_bar = full_bar + kPairStages;      // each CTA its own: "my stage may be refilled"
  uint64_t* acc_full = empty_bar + kPairStages;      // [2] each CTA its own: tensor core -> epilogue
  uint64_t* acc_empty = acc_full + 2;                // [2] leader's only: epilogue warps of BOTH CTAs -> tensor core
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();           // 0: leader (issues the MMAs), 1: peer
  constexpr int BN = kPairBN;

  // Grouped raster over pair tiles: 8 pair-rows share their B panels in L2 while they sweep the tile columns.
  const int tiles_m = (prob.M + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (prob.N + BN - 1) / BN;
  constexpr int kGroup = 8;
  int tile_m, tile_n;
  {
    const int pair = blockIdx.x >> 1;
    const int per_group = kGroup * tiles_n;
    const int group = pair / per_group;
    const int first_m = group * kGroup;
    const int rows_in_group = min(kGroup, tiles_m - first_m);
    const int within = pair % per_group;
    tile_m = first_m + within % rows_in_group;
    tile_n = within / rows_in_group;
  }
  const int pair_m0 = tile_m * 2 * kBM;
  const int m0 = pair_m0 + static_cast<int>(cta) * kBM;      // this CTA's rows of the result
  const int n0 = tile_n * BN;
  const int b_row0 = n0 + static_cast<int>(cta) * (BN / 2);  // this CTA's half of the B tile
  // Symmetric products: pair tiles strictly above the diagonal are produced by mirroring (same decision in both CTAs).
  if (prob.symmetric && global_col(prob, n0) > global_row(prob, min(pair_m0 + 2 * kBM, prob.M) - 1)) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&maps.a_hi);
    tma_prefetch_descriptor(&maps.a_lo);
    tma_prefetch_descriptor(&maps.b_hi);
    tma_prefetch_descriptor(&maps.b_lo);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int k_blocks = (prob.K + kBK - 1) / kBK;
  const int chunks = (k_blocks + kPromote - 1) / kPromote;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer (each CTA loads its own tiles; the bytes are credited to the leader's barrier) ----------------
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int s = kb % kPairStages;
      const uint32_t round = kb / kPairStages;
      if (kb >= kPairStages &&
          !mbar_wait_bounded(&empty_bar[s], (round - 1) & 1, abort_flag, status, kStatusSlotWaitTimeout))
        break;
      uint8_t* stage = smem + s * kPairStageBytes;
      if (cta == 0) mbar_expect_tx(&full_bar[s], 2 * kPairStageBytes);
      const uint32_t leader_bar = map_to_cta(smem_u32(&full_bar[s]), 0);
      const int k0 = kb * kBK;
      const int k2 = MIXED ? 2 * k0 : k0;        // the interleaved bf16 plane has 64 elements per 32 of K
      tma_load_2d_pair(stage, &maps.a_hi, leader_bar, k0, m0);
      tma_load_2d_pair(stage + kBM * kRowBytes, &maps.a_lo, leader_bar, k2, m0);
      tma_load_2d_pair(stage + 2 * kBM * kRowBytes, &maps.b_hi, leader_bar, k0, b_row0);
      tma_load_2d_pair(stage + 2 * kBM * kRowBytes + (BN / 2) * kRowBytes, &maps.b_lo, leader_bar, k2, b_row0);
    }
    if (*abort_flag) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1 && lane == 0 && cta == 0) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    constexpr uint32_t idesc = umma_idesc_tf32(2 * kBM, BN);
    constexpr uint32_t idesc16 = umma_idesc_bf16(2 * kBM, BN);
    bool ok = true;
    int kb = 0;
    for (int c = 0; c < chunks && ok; ++c) {
      const int buf = c & 1;
      if (c >= 2) {
        ok = mbar_wait_bounded(&acc_empty[buf], ((c >> 1) - 1) & 1, abort_flag, status, kStatusAccumWaitTimeout);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(buf * BN);
      const int kb_end = min(k_blocks, kb + kPromote);
      for (int first = 1; kb < kb_end; ++kb) {
        const int s = kb % kPairStages;
        const uint32_t round = kb / kPairStages;
        ok = mbar_wait_bounded(&full_bar[s], round & 1, abort_flag, status, kStatusTmaWaitTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t stage = smem_u32(smem + s * kPairStageBytes);
        const uint64_t a_hi = umma_desc_kmajor<kRowBytes>(stage);
        const uint64_t a_2 = umma_desc_kmajor<kRowBytes>(stage + kBM * kRowBytes);
        const uint64_t b_hi = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes);
        const uint64_t b_2 = umma_desc_kmajor<kRowBytes>(stage + 2 * kBM * kRowBytes + (BN / 2) * kRowBytes);
        if constexpr (MIXED) {
          constexpr uint64_t kLb = 64 >> 4;
          const bool tf32_first = (kb & 1) != 0;     // one change of MMA kind per k-block, as in the single-CTA kernel
          if (tf32_first) {
#pragma unroll
            for (int k = 0; k < kBK / 8; ++k) {
              const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
              umma_tf32_ss_pair(tmem_acc, a_hi + adv, b_hi + adv, idesc, first ? 0u : 1u);
              first = 0;
            }
          }
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
            umma_bf16_ss_pair(tmem_acc, a_2 + kLb + adv, b_2 + adv, idesc16, first ? 0u : 1u);     // lo * hi
            first = 0;
            umma_bf16_ss_pair(tmem_acc, a_2 + adv, b_2 + kLb + adv, idesc16, 1);                   // hi * lo
          }
          if (!tf32_first) {
#pragma unroll
            for (int k = 0; k < kBK / 8; ++k) {
              const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
              umma_tf32_ss_pair(tmem_acc, a_hi + adv, b_hi + adv, idesc, 1);
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < kBK / 8; ++k) {
            const uint64_t adv = static_cast<uint64_t>(k * 32 >> 4);
            umma_tf32_ss_pair(tmem_acc, a_2 + adv, b_hi + adv, idesc, first ? 0u : 1u);
            first = 0;
            umma_tf32_ss_pair(tmem_acc, a_hi + adv, b_2 + adv, idesc, 1);
            umma_tf32_ss_pair(tmem_acc, a_hi + adv, b_hi + adv, idesc, 1);
          }
        }
        umma_commit_pair(&empty_bar[s]);  // both CTAs' stage s may be refilled once these UMMAs have read it
      }
      if (ok) umma_commit_pair(&acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ---------------- promotion + epilogue (each CTA its own 128 rows) ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    constexpr int kCols = BN / 2;
    const int col0 = half * kCols;
    const uint32_t leader_acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    float sum[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) sum[j] = 0.0f;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int buf = c & 1;
      ok = mbar_wait_bounded(&acc_full[buf], (c >> 1) & 1, abort_flag, status, kStatusAccumWaitTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * BN + col0);
#pragma unroll
      for (int cc = 0; cc < kCols; cc += 32) {
        uint32_t raw[32];
        tmem_ld_32x32(taddr + static_cast<uint32_t>(cc), raw);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[cc + j] += __uint_as_float(raw[j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + static_cast<uint32_t>(buf * sizeof(uint64_t)));
    }
    float* tile = reinterpret_cast<float*>(smem);
    {
      const int m_local = quarter * 32 + lane;
#pragma unroll
      for (int jx = 0; jx < kCols; ++jx) tile[(col0 + jx) * kTilePitch + m_local] = sum[jx];
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kEpiWarps * 32) : "memory");
    if (ok && m0 < prob.M) run_epilogue<BN, MODE>(prob, tile, m0, n0, ew, lane, 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                 // nobody leaves while the other CTA may still touch its shared memory or TMEM
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps (driver entry point fetched at run time, so no link-time libcuda) and launch.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || ptr == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// K-contiguous fp32 matrix [rows][K] with row pitch ld (floats); box = 32 floats x box_rows rows.
CUtensorMap make_operand_map(const float* base, int64_t K, int64_t rows, int64_t ld, int box_rows) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::invalid_argument("operand plane must be 16-byte aligned");
  if ((ld * 4) % 16 != 0) throw std::invalid_argument("operand plane pitch must be a multiple of 4 floats");
  CUtensorMap map;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem[2] = {1, 1};
  CUresult res = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
                                   elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   kRowBytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(res));
  return map;
}

// Interleaved bf16 plane of a K-contiguous operand: [rows][64 * ceil(K / 32)] elements with row pitch ld
// (elements); box = 64 elements (128 bytes: hb and lb of one 32-element k-block) x box_rows rows.
CUtensorMap make_bf16_map(const uint16_t* base, int64_t K, int64_t rows, int64_t ld, int box_rows) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::invalid_argument("bf16 operand plane must be 16-byte aligned");
  const int64_t extent = 64 * ((K + 31) / 32);
  if (ld % 64 != 0 || ld < extent) throw std::invalid_argument("bf16 operand plane pitch must be a multiple of 64 elements covering K");
  CUtensorMap map;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(extent), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(2 * kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem[2] = {1, 1};
  CUresult res = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(base), dims, strides, box,
                                   elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (bf16) failed with code " + std::to_string(res));
  return map;
}

template <int BN, int MODE, bool MIXED>
void launch(const GemmOperands& ops, const GemmProblem& prob, int* status, cudaStream_t stream) {
  using Cfg = TileConfig<BN>;
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(gemm_tf32x3_kernel<BN, MODE, MIXED>), Cfg::kSmemBytes, configured, "gemm_tf32x3");
  GemmMaps maps;
  const int64_t a_k = ops.a_k_total ? ops.a_k_total : prob.K, a_rows = ops.a_rows_total ? ops.a_rows_total : prob.M;
  const int64_t b_k = ops.b_k_total ? ops.b_k_total : prob.K, b_rows = ops.b_rows_total ? ops.b_rows_total : prob.N;
  maps.a_hi = make_operand_map(ops.a_hi, a_k, a_rows, ops.lda, kBM);
  maps.b_hi = make_operand_map(ops.b_hi, b_k, b_rows, ops.ldb, BN);
  if constexpr (MIXED) {
    maps.a_lo = make_bf16_map(ops.a_hl, a_k, a_rows, ops.lda16, kBM);
    maps.b_lo = make_bf16_map(ops.b_hl, b_k, b_rows, ops.ldb16, BN);
  } else {
    maps.a_lo = make_operand_map(ops.a_lo, a_k, a_rows, ops.lda, kBM);
    maps.b_lo = make_operand_map(ops.b_lo, b_k, b_rows, ops.ldb, BN);
  }
  const int tiles_m = (prob.M + kBM - 1) / kBM;
  const int tiles_n = (prob.N + BN - 1) / BN;
  const int splits = (MODE == kEpiStore && prob.k_splits > 1) ? prob.k_splits : 1;
  dim3 grid(tiles_m * tiles_n, splits, prob.batches > 1 ? prob.batches : 1);
  gemm_tf32x3_kernel<BN, MODE, MIXED><<<grid, kThreads, Cfg::kSmemBytes, stream>>>(maps, prob, status);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("gemm_tf32x3 launch: ") + cudaGetErrorString(err));
}

template <int MODE, bool MIXED>
void launch_pair(const GemmOperands& ops, const GemmProblem& prob, int* status, cudaStream_t stream) {
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(gemm_pair_kernel<MODE, MIXED>), kPairSmemBytes, configured, "gemm_pair");
  GemmMaps maps;
  const int64_t a_k = ops.a_k_total ? ops.a_k_total : prob.K, a_rows = ops.a_rows_total ? ops.a_rows_total : prob.M;
  const int64_t b_k = ops.b_k_total ? ops.b_k_total : prob.K, b_rows = ops.b_rows_total ? ops.b_rows_total : prob.N;
  maps.a_hi = make_operand_map(ops.a_hi, a_k, a_rows, ops.lda, kBM);
  maps.b_hi = make_operand_map(ops.b_hi, b_k, b_rows, ops.ldb, kPairBN / 2);
  if constexpr (MIXED) {
    maps.a_lo = make_bf16_map(ops.a_hl, a_k, a_rows, ops.lda16, kBM);
    maps.b_lo = make_bf16_map(ops.b_hl, b_k, b_rows, ops.ldb16, kPairBN / 2);
  } else {
    maps.a_lo = make_operand_map(ops.a_lo, a_k, a_rows, ops.lda, kBM);
    maps.b_lo = make_operand_map(ops.b_lo, b_k, b_rows, ops.ldb, kPairBN / 2);
  }
  const int tiles_m = (prob.M + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (prob.N + kPairBN - 1) / kPairBN;
  dim3 grid(2 * tiles_m * tiles_n, 1, 1);
  gemm_pair_kernel<MODE, MIXED><<<grid, kThreads, kPairSmemBytes, stream>>>(maps, prob, status);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string("gemm_pair launch: ") + cudaGetErrorString(err));
}

bool g_use_pairs = true;

}  // namespace

void gemm_use_cta_pairs(bool on) { g_use_pairs = on; }

void gemm_tf32x3(const GemmOperands& ops, const GemmProblem& prob, int* status, cudaStream_t stream) {
  if (prob.M <= 0 || prob.N <= 0) return;
  if (prob.mode == kEpiPush && (prob.push_table == nullptr || prob.push_nb < 1 || prob.push_Pr < 1 || prob.push_Pc < 1 ||
                                prob.k_splits > 1 || prob.batches > 1 || prob.symmetric))
    throw std::invalid_argument("gemm_tf32x3: the push epilogue needs a target table and a plain (unsplit, unbatched) product");
  if (prob.K <= 0) throw std::invalid_argument("gemm_tf32x3 needs K >= 1");
  // Wide tiles when there are enough of them to fill the 148 SMs; narrower tiles otherwise.
  const int64_t wide_tiles = static_cast<int64_t>((prob.M + kBM - 1) / kBM) * ((prob.N + 255) / 256);
  const bool wide = prob.N > 128 && wide_tiles >= 148 && !prob.force_narrow;
  const bool mixed = ops.a_hl && ops.b_hl;
  if (mixed && kBK != 32) throw std::invalid_argument("gemm_tf32x3: mixed corrections need the 32-element k-block build");
#define SOAP_GEMM_LAUNCH(MODE_)                                                                      \
  do {                                                                                               \
    if (mixed) {                                                                                     \
      wide ? launch<256, MODE_, true>(ops, prob, status, stream) : launch<128, MODE_, true>(ops, prob, status, stream);   \
    } else {                                                                                         \
      wide ? launch<256, MODE_, false>(ops, prob, status, stream) : launch<128, MODE_, false>(ops, prob, status, stream); \
    }                                                                                                \
  } while (0)
  // CTA pairs for large plain problems: no batching, no split-K
  const bool pairs = g_use_pairs && wide && kBK == 32 && prob.M >= 2 * kBM && prob.batches <= 1 && prob.k_splits <= 1 &&
                     prob.mode != kEpiPairUpdate;
  if (pairs) {
#define SOAP_PAIR_LAUNCH(MODE_)                                                                                  \
  do {                                                                                                           \
    if (mixed) launch_pair<MODE_, true>(ops, prob, status, stream); else launch_pair<MODE_, false>(ops, prob, status, stream); \
  } while (0)
    switch (prob.mode) {
      case kEpiStore: SOAP_PAIR_LAUNCH(kEpiStore); return;
      case kEpiSplit: SOAP_PAIR_LAUNCH(kEpiSplit); return;
      case kEpiAdam: SOAP_PAIR_LAUNCH(kEpiAdam); return;
      case kEpiRowMajor: SOAP_PAIR_LAUNCH(kEpiRowMajor); return;
      case kEpiPush: SOAP_PAIR_LAUNCH(kEpiPush); return;
      default: break;
    }
#undef SOAP_PAIR_LAUNCH
  }
  switch (prob.mode) {
    case kEpiStore:
      SOAP_GEMM_LAUNCH(kEpiStore);
      break;
    case kEpiSplit:
      SOAP_GEMM_LAUNCH(kEpiSplit);
      break;
    case kEpiAdam:
      SOAP_GEMM_LAUNCH(kEpiAdam);
      break;
    case kEpiRowMajor:
      SOAP_GEMM_LAUNCH(kEpiRowMajor);
      break;
    case kEpiPush:
      SOAP_GEMM_LAUNCH(kEpiPush);
      break;
    case kEpiPairUpdate:
      if (prob.N != 128 || prob.remap == nullptr || prob.Chi == nullptr)
        throw std::invalid_argument("gemm_tf32x3: the pair update needs N = 128, a remap table and output planes");
      if (mixed) throw std::invalid_argument("gemm_tf32x3: the pair update takes fp32 planes only");
      launch<128, kEpiPairUpdate, false>(ops, prob, status, stream);
      break;
    default:
      throw std::invalid_argument("gemm_tf32x3: unknown epilogue mode");
  }
#undef SOAP_GEMM_LAUNCH
}

}  // namespace soapb200
