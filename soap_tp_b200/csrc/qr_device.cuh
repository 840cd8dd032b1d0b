// Device-side pieces shared by the panel factorisation kernels (qr.cu, qr_panel_pairs.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "launch_util.h"
#include "qr.h"
#include "status.h"

namespace soapb200 {

// Sequence base of the next panel launch.  One counter for both panel kernels: they may be handed the
// same exchange buffer with different slot layouts, and a sequence number used by one must never be
// accepted by the other on a stale word.
unsigned int next_panel_epoch();

namespace qrdev {

constexpr int kB = kQrPanelWidth;
constexpr int kRows = kQrRowsPerCta;
constexpr int kPanelThreads = 512;
constexpr int kPitch = kB + 1;


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
  long long* trace;              // optional diagnostics output, may be null: the pair kernel stores its number of
                                 // exchange steps; the one-column kernel stores clock64 stamps of CTA 0 at column 64
                                 // when it is compiled with SOAP_QR_TRACE
  int debug_skip;                // SOAP_QR_TRACE builds only: bit 0 skips the T column, bit 1 the pivot-row bookkeeping
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

// Column cc of the compact-WY factor: T[0:cc, cc] = -tau_cc * T[0:cc, 0:cc] * S[0:cc, cc], T[cc, cc] = tau_cc.
// Called by all 512 threads of a CTA: four threads share a row, two independent accumulators each.
__device__ __forceinline__ void t_column(float (*T)[kPitch], const float* scol, const float* taus, int cc, int t) {
  const int i = t >> 2, part = t & 3;
  float a0 = 0.f, a1 = 0.f;
  if (i < cc) {
    int k = i + part;
    for (; k + 4 < cc; k += 8) {
      a0 = fmaf(T[i][k], scol[k], a0);
      a1 = fmaf(T[i][k + 4], scol[k + 4], a1);
    }
    if (k < cc) a0 = fmaf(T[i][k], scol[k], a0);
  }
  float acc = a0 + a1;
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  if (part == 0) {
    if (i < cc) T[i][cc] = -taus[cc] * acc;
    else if (i == cc) T[i][cc] = taus[cc];
  }
}


}  // namespace qrdev
}  // namespace soapb200
